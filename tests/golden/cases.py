"""Seeded input generators shared by the golden-vector generator and the parity tests.

Every case is a function of its name only: the same torch version and seed give the same
tensors on any machine, so a fixture generated where the reference implementation is
importable can be checked on a machine where it is not.

A case is a dict with
  ``tensors``  ordered ``{fqn: torch.Tensor}`` (CPU; may be views / non-contiguous),
  ``blobs``    ordered ``{fqn: bytes}`` for the BYTE_IO path,
  ``bucket_count`` the writer thread / object count passed to ``prepare_write_data``.
"""

from __future__ import annotations

import io
from typing import Callable, Dict

import torch

FLOAT_DTYPES = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
INT_DTYPES = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def _rand(g: torch.Generator, shape, dtype: torch.dtype) -> torch.Tensor:
    """Random tensor whose every byte is exercised (no all-zero payloads)."""
    if dtype == torch.bool:
        return torch.randint(0, 2, shape, generator=g, dtype=torch.uint8).to(torch.bool)
    if dtype in (torch.complex64, torch.complex128):
        real = torch.float32 if dtype == torch.complex64 else torch.float64
        return torch.complex(torch.randn(shape, generator=g, dtype=real), torch.randn(shape, generator=g, dtype=real))
    if dtype.is_floating_point:
        return torch.randn(shape, generator=g, dtype=torch.float32).to(dtype)
    info = torch.iinfo(dtype)
    hi = min(info.max, 2**31 - 1)
    lo = max(info.min, -(2**31))
    return torch.randint(lo, hi, shape, generator=g, dtype=torch.int64).to(dtype)


def case_mixed() -> dict:
    """Every dtype the reference's own save tests walk, odd lengths, 0-dim, empty, up to 4-D."""
    g = _gen(101)
    t: Dict[str, torch.Tensor] = {}
    shapes = [(), (1,), (3,), (17,), (257,), (5, 7), (2, 3, 5), (2, 3, 4, 5), (0,), (4, 0, 3), (1023,), (64, 33)]
    dtypes = FLOAT_DTYPES + INT_DTYPES + (torch.bool, torch.complex64)
    k = 0
    for si, shape in enumerate(shapes):
        for di, dtype in enumerate(dtypes):
            # not the full cross product: a diagonal band keeps the fixture small
            if (si + di) % 3 != 0:
                continue
            t[f"m.{k}.{str(dtype).split('.')[-1]}"] = _rand(g, shape, dtype)
            k += 1
    blobs = {
        "extra.rng": bytes(range(256)) * 3 + b"\x00\x01",
        "extra.empty": b"",
        "extra.cfg": b"{'a': 1, 'b': [1, 2, 3]}" * 11,
    }
    return {"tensors": t, "blobs": blobs, "bucket_count": 1}


def case_views() -> dict:
    """Non-contiguous sources: transposes, permutes, slices with storage offsets, steps, expands."""
    g = _gen(202)
    t: Dict[str, torch.Tensor] = {}
    base = _rand(g, (37, 53), torch.float32)
    t["v.t2d.f32"] = base.t()
    t["v.t2d.bf16"] = _rand(g, (96, 40), torch.bfloat16).t()
    t["v.t2d.i64"] = _rand(g, (19, 33), torch.int64).t()
    t["v.t2d.u8"] = _rand(g, (70, 45), torch.uint8).t()
    t["v.rowslice"] = base[5:20]  # contiguous, storage offset != 0
    t["v.colslice"] = base[:, 3:29]  # inner-contiguous rows with a gap
    t["v.step"] = base[::2, ::3]
    t["v.perm3"] = _rand(g, (6, 10, 14), torch.float16).permute(2, 0, 1)
    t["v.perm4"] = _rand(g, (3, 4, 5, 6), torch.float32).permute(0, 3, 1, 2)
    t["v.swap_outer"] = _rand(g, (5, 7, 16), torch.bfloat16).transpose(0, 1)
    t["v.expand"] = _rand(g, (1, 9), torch.int32).expand(4, 9)
    t["v.odd_offset_1d"] = _rand(g, (1001,), torch.int16)[1:]
    t["v.scalar_view"] = base[3, 4]
    t["v.narrow_bytes"] = _rand(g, (333,), torch.uint8)[7:300]
    t["v.f64_t"] = _rand(g, (11, 13), torch.float64).t()
    return {"tensors": t, "blobs": {}, "bucket_count": 1}


def case_two_buckets() -> dict:
    """bucket_count=2: tensors are greedily binned largest first, blobs round-robin."""
    g = _gen(303)
    t: Dict[str, torch.Tensor] = {}
    sizes = [(128, 64), (10,), (77, 3), (4096,), (33, 33), (2, 2), (513,), (9, 9, 9)]
    for i, s in enumerate(sizes):
        dt = (torch.float32, torch.bfloat16, torch.int64)[i % 3]
        t[f"b.{i}"] = _rand(g, s, dt)
    blobs = {"blob.0": b"zero" * 5, "blob.1": b"one" * 7, "blob.2": b"two" * 9}
    return {"tensors": t, "blobs": blobs, "bucket_count": 2}


def case_gpt2_tiny() -> dict:
    """GPT-2-shaped state dict (tied embedding, LayerNorm gains 1.0) + Adam state, scaled down.

    2 layers, d_model 48, d_ff 192, vocab 211, ctx 32. Value distributions follow the full-size
    configuration: weights N(0, 0.02), exp_avg N(0, 1e-3), exp_avg_sq its square, step = 1000.
    """
    g = _gen(0)
    d, ff, vocab, ctx, layers = 48, 192, 211, 32, 2
    p: Dict[str, torch.Tensor] = {}

    def w(*shape):
        return torch.randn(shape, generator=g, dtype=torch.float32) * 0.02

    p["wte.weight"] = w(vocab, d)
    p["wpe.weight"] = w(ctx, d)
    for i in range(layers):
        pre = f"h.{i}."
        p[pre + "ln_1.weight"] = torch.ones(d)
        p[pre + "ln_1.bias"] = torch.zeros(d)
        p[pre + "attn.c_attn.weight"] = w(d, 3 * d)
        p[pre + "attn.c_attn.bias"] = torch.zeros(3 * d)
        p[pre + "attn.c_proj.weight"] = w(d, d)
        p[pre + "attn.c_proj.bias"] = torch.zeros(d)
        p[pre + "ln_2.weight"] = torch.ones(d)
        p[pre + "ln_2.bias"] = torch.zeros(d)
        p[pre + "mlp.c_fc.weight"] = w(d, ff)
        p[pre + "mlp.c_fc.bias"] = torch.zeros(ff)
        p[pre + "mlp.c_proj.weight"] = w(ff, d)
        p[pre + "mlp.c_proj.bias"] = torch.zeros(d)
    p["ln_f.weight"] = torch.ones(d)
    p["ln_f.bias"] = torch.zeros(d)
    t: Dict[str, torch.Tensor] = {}
    for k, v in p.items():
        t["model." + k] = v
    for k, v in p.items():
        m = torch.randn(v.shape, generator=g, dtype=torch.float32) * 1e-3
        t[f"optim.state.{k}.exp_avg"] = m
        t[f"optim.state.{k}.exp_avg_sq"] = (torch.randn(v.shape, generator=g, dtype=torch.float32) * 1e-3) ** 2
        t[f"optim.state.{k}.step"] = torch.tensor(1000, dtype=torch.int64)
    return {"tensors": t, "blobs": {"optim.param_groups": b"\x80\x04]\x94."}, "bucket_count": 1}


CASES: Dict[str, Callable[[], dict]] = {
    "mixed": case_mixed,
    "views": case_views,
    "two_buckets": case_two_buckets,
    "gpt2_tiny": case_gpt2_tiny,
}

# (dtype, shape) pairs whose pickled header bytes are pinned one by one.
HEADER_MATRIX = [
    (dt, sh)
    for dt in FLOAT_DTYPES + INT_DTYPES + (torch.bool, torch.complex64, torch.complex128)
    for sh in [(), (0,), (1,), (255,), (256,), (65535,), (65536,), (4096, 14336), (2, 3, 4), (1, 2, 3, 4), (2, 1, 2, 1, 2), (2**31,), (2**31 - 1, 1)]
]

# Sub-block reads of a saved tensor: (saved shape, dtype, storage_offsets, lengths).
NARROW_CASES = [
    ((16, 24), torch.float32, (0, 0), (16, 24)),
    ((16, 24), torch.float32, (4, 0), (8, 24)),
    ((16, 24), torch.bfloat16, (0, 5), (16, 7)),
    ((16, 24), torch.int64, (3, 9), (5, 11)),
    ((6, 5, 8), torch.float16, (1, 2, 3), (4, 2, 5)),
    ((4, 3, 5, 7), torch.uint8, (0, 1, 0, 2), (4, 2, 5, 3)),
    ((129,), torch.bfloat16, (17,), (100,)),
    ((), torch.int64, (), ()),
]


def narrow_source(i: int) -> torch.Tensor:
    shape, dtype, _, _ = NARROW_CASES[i]
    return _rand(_gen(900 + i), shape, dtype)


def write_items_and_resolver(case: dict):
    """Builds DCP ``WriteItem``s (default-planner style) and a resolver for a case."""
    from torch.distributed.checkpoint.planner_helpers import _create_write_items

    lookup = {}
    items = []
    for fqn, tensor in case["tensors"].items():
        items.extend(_create_write_items(fqn, tensor))
        lookup[fqn] = tensor
    for fqn, blob in case["blobs"].items():
        items.extend(_create_write_items(fqn, blob))
        lookup[fqn] = blob

    class _Resolver:
        def resolve_data(self, write_item):
            obj = lookup[write_item.index.fqn]
            if isinstance(obj, bytes):
                return io.BytesIO(obj)
            return obj

    return items, _Resolver()
