"""Compile a ``RoutingTable`` into flat copy descriptors and execute them.

A descriptor is one strided 2-D slice copy from the sending rank's flat parameter buffer into a
destination rank's flat buffer. For every routed (actor shard, sampler shard) pair the compiler
intersects the two shards' boxes in full-parameter coordinates (so TP re-slicing, the QKV
group-interleave, the gate/up halves and per-expert slices all reduce to box intersections) and emits
one descriptor per non-empty intersection. ``execute_plan`` runs the whole list in ONE native kernel
launch over NVLink peer pointers (optionally quantising to block-scaled fp8 on the way); on CPU
tensors it applies the same descriptors with plain slicing, which is the oracle the tests compare
against "gather the full tensor, then slice for the sampler".
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np
import torch

from .routing_table import RoutingTable

DESC_DTYPE = np.dtype([("src_off", "<i8"), ("dst_off", "<i8"), ("rows", "<i4"), ("cols", "<i4"),
                       ("src_stride", "<i8"), ("dst_stride", "<i8"), ("dst_rank", "<i4"), ("quant", "<i4"),
                       ("dst_scale_off", "<i8"), ("scale_cols", "<i4"), ("pad", "<i4")])
assert DESC_DTYPE.itemsize == 64


def _box_offsets(boxes):
    """Start offset of every box inside the shard's local storage (boxes stored one after another)."""
    offs, acc = [], 0
    for r0, r1, c0, c1 in boxes:
        offs.append(acc)
        acc += (r1 - r0) * (c1 - c0)
    return offs


@dataclass
class SyncPlan:
    descs: np.ndarray            # DESC_DTYPE [n]
    work_prefix: np.ndarray      # int64 [n]: first 16-byte work item of each descriptor
    total_work: int
    total_bytes: int
    _dev: dict | None = None

    def to_device(self, device):
        if self._dev is None or self._dev["device"] != device:
            self._dev = {"device": device,
                         "descs": torch.from_numpy(self.descs.view(np.uint8).copy()).to(device),
                         "prefix": torch.from_numpy(self.work_prefix.copy()).to(device)}
        return self._dev


def compile_plan(table: RoutingTable, actor_rank: int, actor_offsets: dict, sampler_offsets: dict,
                 sampler_scale_offsets: dict | None = None, quant: bool = False, elem_bytes: int = 2) -> SyncPlan:
    """``actor_offsets[name]`` / ``sampler_offsets[rank][name]``: element offset of the parameter's shard
    inside that rank's flat buffer. With ``quant`` 2-D matrices become fp8 bytes + fp32 block scales at
    ``sampler_scale_offsets[rank][name]`` (1-D tensors are still copied as bf16 and must live in a bf16
    region of the destination)."""
    rows = []
    for s_rank, items in sorted(table.get_transfers_for_actor_rank(actor_rank).items()):
        for it in items:
            a, s = it["actor"], it["sampler"]
            ab, sb = a.metadata["boxes"], s.metadata["boxes"]
            ao, so = _box_offsets(ab), _box_offsets(sb)
            a_base, s_base = actor_offsets[a.param_name], sampler_offsets[s_rank][s.param_name]
            q = 1 if (quant and len(s.full_param_shape) >= 2) else 0
            s_cols_total = sb[0][3] - sb[0][2]
            for (ar0, ar1, ac0, ac1), aoff in zip(ab, ao):
                for (sr0, sr1, sc0, sc1), soff in zip(sb, so):
                    r0, r1, c0, c1 = max(ar0, sr0), min(ar1, sr1), max(ac0, sc0), min(ac1, sc1)
                    if r0 >= r1 or c0 >= c1:
                        continue
                    aw, sw = ac1 - ac0, sc1 - sc0
                    d = np.zeros((), dtype=DESC_DTYPE)
                    d["src_off"] = a_base + aoff + (r0 - ar0) * aw + (c0 - ac0)
                    d["dst_off"] = s_base + soff + (r0 - sr0) * sw + (c0 - sc0)
                    d["rows"], d["cols"], d["src_stride"], d["dst_stride"] = r1 - r0, c1 - c0, aw, sw
                    d["dst_rank"], d["quant"] = s_rank, q
                    if q:
                        assert (r0 - sr0) % 128 == 0 and (c0 - sc0) % 128 == 0 and soff % 128 == 0, \
                            "fp8 sync needs 128-aligned slices"
                        sc_cols = (s_cols_total + 127) // 128
                        local_row0 = soff // sw + (r0 - sr0)
                        d["dst_scale_off"] = sampler_scale_offsets[s_rank][s.param_name] + (local_row0 // 128) * sc_cols + (c0 - sc0) // 128
                        d["scale_cols"] = sc_cols
                    rows.append(d)
    return plan_from_descs(rows, elem_bytes)


def copy_desc(src_off: int, dst_off: int, rows: int, cols: int, src_stride: int, dst_stride: int, dst_rank: int):
    """One bf16 slice copy: ``rows x cols`` elements from ``src_off`` (row stride ``src_stride``) of the
    sender's buffer to ``dst_off`` of rank ``dst_rank``'s buffer. Offsets and strides are multiples of
    8 elements (16-byte vectors)."""
    d = np.zeros((), dtype=DESC_DTYPE)
    d["src_off"], d["dst_off"], d["rows"], d["cols"] = src_off, dst_off, rows, cols
    d["src_stride"], d["dst_stride"], d["dst_rank"] = src_stride, dst_stride, dst_rank
    return d


def plan_from_descs(rows: list, elem_bytes: int = 2) -> SyncPlan:
    descs = np.array(rows, dtype=DESC_DTYPE) if rows else np.zeros(0, dtype=DESC_DTYPE)
    per = descs["rows"].astype(np.int64) * ((descs["cols"].astype(np.int64) + 7) // 8)
    prefix = np.concatenate([[0], np.cumsum(per)[:-1]]).astype(np.int64) if len(descs) else np.zeros(0, np.int64)
    nbytes = int((descs["rows"].astype(np.int64) * descs["cols"]).sum()) * elem_bytes
    return SyncPlan(descs, prefix, int(per.sum()), nbytes)


def fp8_block_quant_ref(x: torch.Tensor):
    """128x128 block quantisation in PyTorch: (fp8 e4m3 tensor, fp32 scales) with scale = amax/448
    (1 where amax is 0 or not finite); dequant = fp8 * scale."""
    R, Cc = x.shape
    br, bc = (R + 127) // 128, (Cc + 127) // 128
    xp = torch.zeros(br * 128, bc * 128, dtype=torch.float32, device=x.device)
    xp[:R, :Cc] = x.float()
    blk = xp.view(br, 128, bc, 128).permute(0, 2, 1, 3)
    amax = blk.abs().amax((-1, -2))
    scale = torch.where((amax > 0) & torch.isfinite(amax), amax / 448.0, torch.ones_like(amax))
    q = (blk / scale[..., None, None]).clamp(-448, 448).permute(0, 2, 1, 3).reshape(br * 128, bc * 128)[:R, :Cc]
    return q.to(torch.float8_e4m3fn), scale


def execute_plan(plan: SyncPlan, src_flat: torch.Tensor, dst_flats: list, dst_ptrs: list[int] | None = None,
                 scale_flats: list | None = None, scale_ptrs: list[int] | None = None) -> None:
    """Run the plan. CUDA: one kernel launch writing through ``dst_ptrs`` (peer pointers, index =
    destination rank; defaults to the data pointers of ``dst_flats``). CPU: slice copies."""
    if len(plan.descs) == 0:
        return
    if not src_flat.is_cuda:
        for d in plan.descs:
            r, c = int(d["rows"]), int(d["cols"])
            src = src_flat[int(d["src_off"]):].as_strided((r, c), (int(d["src_stride"]), 1))
            dst_buf = dst_flats[int(d["dst_rank"])]
            if d["quant"]:
                q, sc = fp8_block_quant_ref(src)
                dst_buf.view(torch.uint8)[int(d["dst_off"]):].as_strided((r, c), (int(d["dst_stride"]), 1)).copy_(q.view(torch.uint8))
                sb = scale_flats[int(d["dst_rank"])]
                sb[int(d["dst_scale_off"]):].as_strided(sc.shape, (int(d["scale_cols"]), 1)).copy_(sc)
            else:
                dst_buf[int(d["dst_off"]):].as_strided((r, c), (int(d["dst_stride"]), 1)).copy_(src)
        return
    from ...ops import _common as C
    lib = C.lib()
    dev = plan.to_device(src_flat.device)
    world = len(dst_ptrs) if dst_ptrs is not None else len(dst_flats)
    ptrs = dst_ptrs if dst_ptrs is not None else [0 if t is None else t.data_ptr() for t in dst_flats]
    arr = (ctypes.c_ulonglong * world)(*ptrs)
    copies = plan.descs["quant"] == 0
    if copies.all():
        rc = lib.axb_p2p_copy_plan(C.ptr(src_flat), arr, world, C.ptr(dev["descs"]), C.ptr(dev["prefix"]),
                                   len(plan.descs), ctypes.c_longlong(plan.total_work), C.stream())
        C.launched(rc, "p2p_copy_plan")
        return
    # mixed plan: bf16 descriptors through the copy kernel, matrices through the quantising kernel
    if "split" not in dev:
        cp = plan.descs[copies]
        per = cp["rows"].astype(np.int64) * ((cp["cols"].astype(np.int64) + 7) // 8)
        qd = plan.descs[~copies]
        tiles = [(i, br, bc, 0) for i, d in enumerate(qd) for br in range((int(d["rows"]) + 127) // 128)
                 for bc in range((int(d["cols"]) + 127) // 128)]
        dev["split"] = dict(
            cp=torch.from_numpy(cp.view(np.uint8).copy()).to(src_flat.device) if len(cp) else None,
            cp_prefix=torch.from_numpy(np.concatenate([[0], np.cumsum(per)[:-1]]).astype(np.int64)).to(src_flat.device) if len(cp) else None,
            cp_n=len(cp), cp_work=int(per.sum()),
            qd=torch.from_numpy(qd.view(np.uint8).copy()).to(src_flat.device),
            tiles=torch.tensor(tiles, dtype=torch.int32, device=src_flat.device), n_tiles=len(tiles))
    sp = dev["split"]
    if sp["cp_n"]:
        rc = lib.axb_p2p_copy_plan(C.ptr(src_flat), arr, world, C.ptr(sp["cp"]), C.ptr(sp["cp_prefix"]), sp["cp_n"],
                                   ctypes.c_longlong(sp["cp_work"]), C.stream())
        C.launched(rc, "p2p_copy_plan")
    sptrs = scale_ptrs if scale_ptrs is not None else [0 if t is None else t.data_ptr() for t in scale_flats]
    sarr = (ctypes.c_ulonglong * world)(*sptrs)
    rc = lib.axb_p2p_quant_plan(C.ptr(src_flat), arr, sarr, world, C.ptr(sp["qd"]), C.ptr(sp["tiles"]), sp["n_tiles"], C.stream())
    C.launched(rc, "p2p_quant_plan")
