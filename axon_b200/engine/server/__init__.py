from .routers import build_engine_app  # noqa: F401
