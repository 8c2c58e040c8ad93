"""Sampler server: runs one ``GenerationEngine`` on its own thread and serves concurrent generation
requests with continuous batching. Callers get futures (in-process) or use the OpenAI-compatible
HTTP routes. Control surface follows the reference's vLLM server wrapper
(axon/sampler/vllm/server.py:379-845, axon/sampler/base/server.py:35-181): ``/v1/completions`` with
prompt token ids in and ``token_ids`` / ``logprobs`` / ``routed_experts`` out, ``/pause_generation``
with strategy ``drain | hold | continue | reset``, ``/continue_generation``, sleep and wake.
"""
from __future__ import annotations

import asyncio
import base64
import queue
import threading
import time
from concurrent.futures import Future
from enum import Enum

import numpy as np

from .params import SamplingParams, TokenOutput


class SamplerMode(Enum):
    HYBRID = "hybrid"          # shares GPUs and weights with the trainer, alternates with it
    COLOCATED = "colocated"    # same node, own GPUs
    STANDALONE = "standalone"  # separate sampler pool (disaggregated)


SERVER_REGISTRY: dict[str, type] = {}


def register_server(name: str):
    def deco(cls):
        SERVER_REGISTRY[name] = cls
        return cls
    return deco


def params_from_dict(d: dict | None, default_max_tokens: int = 1024) -> SamplingParams:
    d = dict(d or {})
    return SamplingParams(
        temperature=float(d.get("temperature", 1.0)), top_k=int(d.get("top_k", 0) or 0) if int(d.get("top_k", 0) or 0) > 0 else 0,
        top_p=float(d.get("top_p", 1.0)), repetition_penalty=float(d.get("repetition_penalty", 1.0)),
        max_tokens=int(d.get("max_tokens", default_max_tokens)), n=int(d.get("n", 1)),
        stop_token_ids=tuple(d.get("stop_token_ids", ()) or ()), ignore_eos=bool(d.get("ignore_eos", False)),
        seed=d.get("seed"))


def encode_routed_experts(rm) -> dict | None:
    """int16 routing record -> {data: base64, shape} (the wire format of ``routed_experts``)."""
    if rm is None:
        return None
    arr = np.asarray(rm, dtype=np.int16)
    return {"data": base64.b64encode(arr.tobytes()).decode("ascii"), "shape": list(arr.shape)}


def decode_routed_experts(obj):
    if not obj:
        return None
    arr = np.frombuffer(base64.b64decode(obj["data"]), dtype=np.int16)
    return arr.reshape(obj["shape"]).copy()


class Lockstep:
    """Control channel of a tensor-parallel sampler group. The engines of the group must take the same requests and
    the same control operations in the same order between the same steps (their collectives pair up step by step),
    so only the group's first rank decides: before every tick that changes anything it sends
    ``{"new": requests, "ops": control operations, "step": run one engine step}`` to the others, which apply it
    and wait for the next message. Sampling needs no exchange: the summed activations are bit-identical on every
    rank, and random draws depend only on (seed, request, position).

    The messages travel over a CPU (gloo) group so that they never queue behind kernels; ``timeout`` is how long a
    follower waits for the next message, so it bounds how long the group may sit idle only through the leader's
    keep-alive messages."""

    def __init__(self, group, keepalive: float = 20.0):
        import torch.distributed as dist
        self.group, self.keepalive = group, keepalive
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.src = dist.get_global_rank(group, 0)
        self.leader = self.rank == 0

    def send(self, msg: dict) -> None:
        import torch.distributed as dist
        dist.broadcast_object_list([msg], src=self.src, group=self.group)

    def recv(self) -> dict:
        import torch.distributed as dist
        box = [None]
        dist.broadcast_object_list(box, src=self.src, group=self.group)
        return box[0]


@register_server("native")
class SamplerServer:
    def __init__(self, engine, tokenizer=None, name: str = "sampler-0", mode: SamplerMode = SamplerMode.HYBRID,
                 lockstep: "Lockstep | None" = None):
        self.engine, self.tokenizer, self.name, self.mode = engine, tokenizer, name, mode
        self.lockstep = lockstep if (lockstep is not None and lockstep.world > 1) else None
        self._ops: "queue.Queue[tuple]" = queue.Queue()
        self._inbox: "queue.Queue[tuple]" = queue.Queue()
        self._futures: dict[int, Future] = {}
        self._thread: threading.Thread | None = None
        self._stop = threading.Event()
        self._wake = threading.Event()
        self._idle = threading.Event()
        self._idle.set()
        self._ctl_lock = threading.Lock()
        self._paused_hold = False
        self.error: BaseException | None = None

    # ------------------------------------------------------------------ lifecycle
    def start(self) -> "SamplerServer":
        if self._thread is None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._loop, daemon=True, name=self.name)
            self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        self._wake.set()
        if self._thread is not None:
            follower = self.lockstep is not None and not self.lockstep.leader
            self._thread.join(timeout=5 if follower else 30)      # a follower ends with the leader's last message
            self._thread = None

    def _loop(self) -> None:
        eng = self.engine
        try:
            if eng.device.type == "cuda":
                import torch
                torch.cuda.set_device(eng.device)
            if self.lockstep is not None and not self.lockstep.leader:
                return self._follow()
            last_sent = time.monotonic()
            while not self._stop.is_set():
                new = self._drain_inbox()
                ops = self._drain_ops()
                busy = eng.has_unfinished() and eng.cache is not None and not self._paused_hold
                if self.lockstep is not None and (new or ops or busy or time.monotonic() - last_sent > self.lockstep.keepalive):
                    self.lockstep.send({"new": new, "ops": [(n, a) for n, a, _ in ops], "step": busy})
                    last_sent = time.monotonic()
                for _, _, done in ops:
                    done.set()
                if busy:
                    self._idle.clear()
                    with self._ctl_lock:
                        eng.step()
                    self._resolve()
                else:
                    self._resolve()
                    self._idle.set()
                    self._wake.wait(0.005)
                    self._wake.clear()
            if self.lockstep is not None:
                self.lockstep.send({"stop": True})
        except BaseException as e:  # noqa: BLE001
            self.error = e
            for f in self._futures.values():
                if not f.done():
                    f.set_exception(e)
            self._futures.clear()
            self._idle.set()
            while True:                          # nobody may wait forever for an operation this thread will not run
                try:
                    self._ops.get_nowait()[2].set()
                except queue.Empty:
                    break

    def _follow(self) -> None:
        """A tensor-parallel follower: apply the leader's messages in order."""
        eng = self.engine
        while True:
            msg = self.lockstep.recv()
            if msg.get("stop"):
                return
            for prompt, params, images in msg.get("new", ()):
                eng.add_request(prompt, params, images) if images else eng.add_request(prompt, params)
            for name, args in msg.get("ops", ()):
                with self._ctl_lock:
                    self._apply_op(name, args)
            if msg.get("step"):
                self._idle.clear()
                with self._ctl_lock:
                    eng.step()
                eng.finished.clear()             # results are delivered by the leader
            else:
                self._idle.set()

    def _drain_inbox(self) -> list:
        """Move queued requests into the engine; returns what a lockstep leader forwards: (prompt, params, images)."""
        taken = []
        while True:
            try:
                prompt, params, fut, images = self._inbox.get_nowait()
            except queue.Empty:
                return taken
            try:
                rid = self.engine.add_request(prompt, params, images) if images else self.engine.add_request(prompt, params)
            except Exception as e:  # noqa: BLE001 - a bad request (e.g. images for a text model) fails alone
                fut.set_exception(e)
                continue
            self._futures[rid] = fut
            taken.append((prompt, params, images))

    # Control operations that change engine state. Alone, a server runs them in the caller's thread; in a lockstep
    # group the leader's loop runs them between two steps and forwards them, so every rank applies them at the same point.
    def _apply_op(self, name: str, args: tuple) -> None:
        eng = self.engine
        if name == "reset":
            eng.pause("reset")
            eng.resume()
        elif name == "sleep":
            eng.sleep()
        elif name == "wake":
            eng.wake_up(*args)
        elif name == "reset_prefix_cache":
            eng.reset_prefix_cache()
        else:
            raise ValueError(f"unknown control operation '{name}'")

    def _drain_ops(self) -> list:
        ops = []
        while True:
            try:
                op = self._ops.get_nowait()
            except queue.Empty:
                return ops
            with self._ctl_lock:
                self._apply_op(op[0], op[1])
            ops.append(op)

    def _run_op(self, name: str, *args, timeout: float = 120.0) -> None:
        if self.lockstep is None:
            with self._ctl_lock:
                self._apply_op(name, args)
            return
        if not self.lockstep.leader:
            return                               # arrives through the leader's message
        done = threading.Event()
        self._ops.put((name, args, done))
        self._wake.set()
        if not done.wait(timeout):
            raise TimeoutError(f"sampler server '{self.name}': control operation '{name}' was not picked up")
        if self.error is not None:
            raise RuntimeError(f"sampler server '{self.name}' has failed") from self.error

    def _resolve(self) -> None:
        fin = self.engine.finished
        for rid in list(fin):
            fut = self._futures.pop(rid, None)
            out = fin.pop(rid)
            if fut is not None and not fut.done():
                fut.set_result(out)

    # ------------------------------------------------------------------ requests
    def submit(self, prompt_ids, params: SamplingParams | dict | None = None, image_data=None) -> Future:
        """``image_data``: vision inputs of the prompt for vision-language models - the processor's output
        (``pixel_values`` + ``image_grid_thw``) or a list of images (PIL, data / file URLs, OpenAI ``image_url`` items)
        that the server's processor turns into it."""
        if self.error is not None:
            raise RuntimeError(f"sampler server '{self.name}' has failed") from self.error
        if not isinstance(params, SamplingParams):
            params = params_from_dict(params)
        fut: Future = Future()
        self._inbox.put((list(prompt_ids), params, fut, self.prepare_images(image_data)))
        self._wake.set()
        return fut

    def prepare_images(self, image_data):
        if not image_data:
            return None
        if isinstance(image_data, dict) and "pixel_values" in image_data:
            import torch
            return {k: torch.as_tensor(v) for k, v in image_data.items() if v is not None}
        proc = getattr(self, "processor", None)
        ip = getattr(proc, "image_processor", None)
        if ip is None:
            raise ValueError("raw images need a processor with an image_processor on the sampler server; send pixel_values + image_grid_thw")
        from ..utils.openai_client import load_images
        out = ip(images=load_images(image_data), return_tensors="pt")
        return {"pixel_values": out["pixel_values"], "image_grid_thw": out["image_grid_thw"]}

    async def generate(self, prompt_ids, params=None, image_data=None) -> TokenOutput:
        return await asyncio.wrap_future(self.submit(prompt_ids, params, image_data))

    def num_pending(self) -> int:
        return len(self._futures) + self._inbox.qsize()

    # ------------------------------------------------------------------ control
    def pause_generation(self, strategy: str = "drain", timeout: float = 600.0) -> None:
        """drain: wait for in-flight requests to finish (new ones queue). hold: freeze in place.
        continue: do nothing (in-flight requests keep running across the weight update).
        reset: abort in-flight requests; they resolve with finish_reason 'abort' and their partial text."""
        if strategy == "continue" or self._follower:
            return
        if strategy == "hold":
            self._paused_hold = True
            self._wait_idle(timeout)
            return
        if strategy == "drain":
            deadline = time.monotonic() + timeout
            while self.num_pending() and time.monotonic() < deadline:
                time.sleep(0.005)
            return
        if strategy == "reset":
            self._run_op("reset")
            self._wake.set()
            return
        raise ValueError(f"unknown pause strategy '{strategy}'")

    def continue_generation(self) -> None:
        self._paused_hold = False
        self._wake.set()

    def _wait_idle(self, timeout: float) -> None:
        self._wake.set()
        self._idle.wait(timeout)

    @property
    def _follower(self) -> bool:
        """A follower of a lockstep group: its engine is driven by the leader's messages, so the control calls
        that reach it directly (the controller addresses every rank) have nothing to do."""
        return self.lockstep is not None and not self.lockstep.leader

    def sleep(self) -> None:
        if self._follower:
            return
        self._paused_hold = True
        self._wait_idle(60.0)
        self._run_op("sleep")

    def wake_up(self, num_pages: int | None = None) -> None:
        self._run_op("wake", num_pages)
        self._paused_hold = False
        self._wake.set()

    def reset_prefix_cache(self) -> None:
        self._run_op("reset_prefix_cache")

    def update_weights(self, named_tensors) -> int:
        """Copy (name, tensor) pairs into the engine's parameter views while generation is held."""
        n = 0
        self.reset_prefix_cache()
        with self._ctl_lock:
            views = self.engine.model.params.views
            hf_views = None
            localize = getattr(self.engine.model, "localize", None)      # a sharded model keeps its part of every tensor
            for name, t in named_tensors:
                if localize is not None:
                    t = localize(name, t)
                    if t is None:
                        continue
                    if isinstance(t, tuple):          # a pipeline stage renumbers its layers: (its own name, tensor)
                        name, t = t
                dst = views.get(name)
                if dst is None:
                    if hf_views is None:
                        hf_views = self.engine.model.params.to_hf_state_dict(export=False)       # views, in this framework's row order
                    dst = hf_views.get(name)
                    if dst is not None and name.rsplit(".", 2)[-2] in ("q_proj", "k_proj"):
                        from ..models.params import _permute_heads, rope_row_perm
                        perm = rope_row_perm(self.engine.model.cfg)
                        if perm is not None:          # checkpoint rotary layout -> kernel layout
                            t = _permute_heads(t, perm, self.engine.model.cfg.head_dim)
                if dst is None:
                    raise KeyError(f"unknown parameter '{name}'")
                dst.copy_(t.to(dst.dtype))
                n += 1
        return n

    # ------------------------------------------------------------------ OpenAI-compatible HTTP app
    def build_app(self):
        from fastapi import FastAPI, HTTPException
        app = FastAPI(title=f"axon_b200 sampler {self.name}")
        server = self

        @app.get("/health")
        async def health():
            return {"status": "ok" if server.error is None else "failed", "pending": server.num_pending()}

        @app.get("/v1/models")
        async def models():
            return {"object": "list", "data": [{"id": server.name, "object": "model"}]}

        @app.post("/v1/completions")
        async def completions(body: dict):
            prompt = body.get("prompt")
            if isinstance(prompt, str):
                if server.tokenizer is None:
                    raise HTTPException(400, "text prompts need a tokenizer; send token ids")
                prompt = server.tokenizer.encode(prompt)
            if not isinstance(prompt, list) or (prompt and not isinstance(prompt[0], int)):
                raise HTTPException(400, "prompt must be a list of token ids")
            n = int(body.get("n", 1))
            try:
                images = server.prepare_images(body.get("image_data"))      # one object: the n samples share the prompt's pages
            except ValueError as e:
                raise HTTPException(400, str(e))
            outs = await asyncio.gather(*(server.generate(prompt, body, images) for _ in range(n)))
            choices = []
            for i, o in enumerate(outs):
                text = server.tokenizer.decode(o.token_ids) if server.tokenizer is not None else ""
                strs = server.tokenizer.token_strs(o.token_ids) if hasattr(server.tokenizer, "token_strs") else []
                choices.append({"index": i, "text": text, "token_ids": o.token_ids, "finish_reason": o.finish_reason,
                                "stop_reason": o.stop_reason,
                                "logprobs": {"token_logprobs": o.logprobs, "tokens": strs},
                                "routed_experts": encode_routed_experts(o.moe_routermap),
                                "spec_decode_metrics": o.spec_decode_metrics.to_dict() if o.spec_decode_metrics is not None else None})
            return {"object": "text_completion", "model": server.name, "choices": choices,
                    "usage": {"prompt_tokens": len(prompt), "completion_tokens": sum(len(o.token_ids) for o in outs)}}

        @app.post("/tokenize")
        async def tokenize(body: dict):
            if server.tokenizer is None:
                raise HTTPException(400, "no tokenizer")
            ids = server.tokenizer.encode(body.get("prompt", ""))
            return {"tokens": ids, "count": len(ids)}

        @app.post("/pause_generation")
        async def pause(body: dict | None = None):
            strategy = (body or {}).get("strategy", "drain")
            await asyncio.get_running_loop().run_in_executor(None, server.pause_generation, strategy)
            return {"status": "paused", "strategy": strategy}

        @app.post("/continue_generation")
        async def cont():
            server.continue_generation()
            return {"status": "running"}

        @app.post("/sleep")
        async def sleep():
            await asyncio.get_running_loop().run_in_executor(None, server.sleep)
            return {"status": "asleep"}

        @app.post("/wake_up")
        async def wake():
            await asyncio.get_running_loop().run_in_executor(None, server.wake_up)
            return {"status": "awake"}

        return app
