"""Ports, addresses and in-thread HTTP serving (reference: axon/utils/networking_utils.py:29-130)."""
from __future__ import annotations

import asyncio
import ipaddress
import socket
import threading


def is_valid_ipv6_address(address: str) -> bool:
    try:
        ipaddress.IPv6Address(address)
        return True
    except ValueError:
        return False


def get_free_port(address: str = "127.0.0.1") -> tuple[int, socket.socket]:
    """Bind an ephemeral port and return it with the still-open socket (close it right before use)."""
    fam = socket.AF_INET6 if is_valid_ipv6_address(address) else socket.AF_INET
    s = socket.socket(fam, socket.SOCK_STREAM)
    s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    s.bind((address, 0))
    return s.getsockname()[1], s


def ensure_port_available(port: int, force: bool = False, address: str = "127.0.0.1") -> None:
    """Raise when something already listens on ``port``. ``force`` is accepted for interface parity;
    this implementation never terminates foreign processes."""
    with socket.socket() as s:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            s.bind((address, port))
        except OSError as e:
            raise RuntimeError(f"port {port} on {address} is in use") from e


def run_uvicorn_in_thread(app, host: str = "127.0.0.1", port: int | None = None, log_level: str = "warning"):
    """Serve ``app`` from a daemon thread. Returns ``(port, server)``; stop with ``server.should_exit = True``."""
    import uvicorn
    if port is None:
        port, sock = get_free_port(host)
        sock.close()
    server = uvicorn.Server(uvicorn.Config(app, host=host, port=port, log_level=log_level))
    threading.Thread(target=server.run, daemon=True, name=f"uvicorn-{port}").start()
    return port, server


async def run_unvicorn(app, server_args=None, server_address: str = "127.0.0.1", max_retries: int = 5):
    """Async variant with retries on port clashes: returns ``(port, serving task)``."""
    import uvicorn
    last = None
    for _ in range(max_retries):
        port, sock = get_free_port(server_address)
        sock.close()
        server = uvicorn.Server(uvicorn.Config(app, host=server_address, port=port, log_level="warning"))
        task = asyncio.create_task(server.serve())
        await asyncio.sleep(0.2)
        if not task.done():
            return port, task
        last = task.exception()
    raise RuntimeError(f"could not start the HTTP server after {max_retries} tries: {last}")
