"""Seeded synthetic state dicts shaped like the benchmark configurations (test-side generators).

No dataset or checkpoint is involved: shapes, dtypes and value distributions follow the
configuration descriptions, values come from a seeded generator.
"""

import io
import math
import pickle

import torch


def packing_microbench(device, count=1024, min_bytes=4 << 10, max_bytes=64 << 20, cap_bytes=8 << 30, seed=1):
    """``count`` tensors, sizes log-uniform in [min, max] (total capped), 50 % bf16 / 40 % fp32 / 10 % int64,
    rank 1-4 with random shapes, 10 % of them transposed (non-contiguous) views."""
    g = torch.Generator().manual_seed(seed)

    def u():
        return float(torch.rand((), generator=g))

    out = {}
    total = 0
    for i in range(count):
        nbytes = int(math.exp(math.log(min_bytes) + u() * (math.log(max_bytes) - math.log(min_bytes))))
        pick = u()
        dtype = torch.bfloat16 if pick < 0.5 else (torch.float32 if pick < 0.9 else torch.int64)
        itemsize = torch.empty((), dtype=dtype).element_size()
        if total + nbytes > cap_bytes:
            nbytes = max(min_bytes, cap_bytes - total)
        numel = max(1, nbytes // itemsize)
        rank = 1 + int(u() * 4)
        transposed = u() < 0.10
        if transposed:
            rank = max(rank, 2)
        dims, rest = [], numel
        for _ in range(rank - 1):
            d = max(1, int(round(math.exp(u() * math.log(max(rest, 1)) / 2))))
            d = min(d, rest)
            dims.append(d)
            rest = max(1, rest // d)
        dims.append(rest)
        if dtype == torch.int64:
            t = torch.randint(0, 2**31, tuple(dims), dtype=torch.int64, device=device)
        else:
            t = torch.randn(tuple(dims), dtype=torch.float32, device=device).to(dtype)
        if transposed:
            t = t.transpose(-1, -2)
        out[f"t{i:04d}"] = t
        total += t.numel() * t.element_size()
        if total >= cap_bytes:
            break
    return out


def moe_expert_parallel_rank(device, rank=0, layers=4, d_model=256, d_ff=896, seed=3):
    """One expert-parallel rank of a Mixtral-shaped model: per layer its expert's three matrices in
    bf16 (on the device), plus the small items that travel with a real checkpoint: RNG state
    bytes, int64 counters (host tensors) and a pickled configuration dictionary."""
    g = torch.Generator().manual_seed(seed * 100 + rank)
    tensors, blobs = {}, {}
    for layer in range(layers):
        p = f"decoder.layers.{layer}.mlp.experts.local_experts.{rank}."
        for name, shape in (("w1", (d_ff, d_model)), ("w3", (d_ff, d_model)), ("w2", (d_model, d_ff))):
            tensors[p + name] = (torch.randn(shape, generator=g) * 0.02).to(torch.bfloat16).to(device)
        tensors[f"decoder.layers.{layer}.router.weight"] = (torch.randn((8, d_model), generator=g) * 0.02).to(torch.bfloat16).to(device)
    tensors["iteration"] = torch.tensor(1000 + rank, dtype=torch.int64)  # host-resident scalars
    tensors["consumed_samples"] = torch.tensor(512000, dtype=torch.int64)
    tensors["cpu_rng_state"] = torch.randint(0, 256, (5056,), generator=g, dtype=torch.uint8)
    blobs["rng.cuda_state"] = bytes(torch.randint(0, 256, (16,), generator=g, dtype=torch.uint8).tolist())
    blobs["rng.python_state"] = pickle.dumps((3, tuple(range(625)), None))
    config = {"num_layers": layers, "hidden_size": d_model, "ffn_hidden_size": d_ff, "num_moe_experts": 8, "moe_router_topk": 2}
    config.update({f"pad_{k}": f"{k:04d}" * 16 for k in range(48)})  # about 4 KB pickled
    blobs["run_config"] = pickle.dumps(config)
    return {"tensors": tensors, "blobs": blobs, "bucket_count": 1}


def tensor_parallel_rank(device, rank=0, tp=8, layers=2, d_model=512, d_ff=1792, vocab=4096, seed=4, as_views=True):
    """One tensor-parallel rank of a Llama-shaped model in bf16: QKV/gate/up split column-wise
    (output dimension), o/down row-wise (input dimension), embeddings on the vocabulary.

    With ``as_views`` the shards are slices of the full matrices (the input-dimension splits are
    then row-sliced views), otherwise each shard is its own contiguous tensor."""
    g = torch.Generator().manual_seed(seed)
    tensors = {}

    def full(*shape):
        return (torch.randn(shape, generator=g) * 0.02).to(torch.bfloat16).to(device)

    def shard(t, dim):
        piece = t.chunk(tp, dim=dim)[rank]
        return piece if as_views else piece.contiguous()

    tensors["embedding.word_embeddings.weight"] = shard(full(vocab, d_model), 0)
    for layer in range(layers):
        p = f"decoder.layers.{layer}."
        tensors[p + "self_attention.linear_qkv.weight"] = shard(full(d_model + 2 * (d_model // 4), d_model), 0)
        tensors[p + "self_attention.linear_proj.weight"] = shard(full(d_model, d_model), 1)
        tensors[p + "mlp.linear_fc1.weight"] = shard(full(2 * d_ff, d_model), 0)
        tensors[p + "mlp.linear_fc2.weight"] = shard(full(d_model, d_ff), 1)
        tensors[p + "input_layernorm.weight"] = torch.ones(d_model, dtype=torch.bfloat16, device=device)
    tensors["output_layer.weight"] = shard(full(vocab, d_model), 0)
    return {"tensors": tensors, "blobs": {}, "bucket_count": 1}


def tensor_parallel_rank_full_size(device, rank=0, tp=8, layers=80, d_model=8192, d_ff=28672, vocab=128256,
                                   heads=64, kv_heads=8, seed=4):
    """One tensor-parallel rank of a Llama-3-70B-shaped model in bf16 at full size (17.6 GB for
    tp=8), drawn directly on the device. Column-wise shards are contiguous; the row-wise ones
    (attention output, MLP down projection) are column slices of wider matrices, i.e. strided rows."""
    g = torch.Generator(device=device).manual_seed(seed * 100 + rank)
    tensors = {}

    def draw(rows, cols):
        return torch.randn((rows, cols), device=device, dtype=torch.bfloat16, generator=g) * 0.02

    def row_sliced(rows, cols):
        return draw(rows, 2 * cols)[:, cols // 2 : cols // 2 + cols]

    qkv_rows = d_model + 2 * (d_model * kv_heads // heads)
    tensors["embedding.word_embeddings.weight"] = draw(vocab // tp, d_model)
    for layer in range(layers):
        p = f"decoder.layers.{layer}."
        tensors[p + "self_attention.linear_qkv.weight"] = draw(qkv_rows // tp, d_model)
        tensors[p + "self_attention.linear_proj.weight"] = row_sliced(d_model, d_model // tp)
        tensors[p + "mlp.linear_fc1.weight"] = draw(2 * d_ff // tp, d_model)
        tensors[p + "mlp.linear_fc2.weight"] = row_sliced(d_model, d_ff // tp)
        tensors[p + "input_layernorm.weight"] = torch.ones(d_model, dtype=torch.bfloat16, device=device)
        tensors[p + "pre_mlp_layernorm.weight"] = torch.ones(d_model, dtype=torch.bfloat16, device=device)
    tensors["decoder.final_layernorm.weight"] = torch.ones(d_model, dtype=torch.bfloat16, device=device)
    tensors["output_layer.weight"] = draw(vocab // tp, d_model)
    return {"tensors": tensors, "blobs": {}, "bucket_count": 1}


def moe_expert_parallel_rank_full_size(device, rank=0, layers=32, d_model=4096, d_ff=14336, seed=3):
    """The expert-parallel rank of ``moe_expert_parallel_rank`` at full size (one expert of
    3 x 14336 x 4096 bf16 per layer, 11.3 GB), expert weights drawn directly on the device; the
    host-resident scalars, RNG state bytes and the pickled configuration are the small generator's."""
    small = moe_expert_parallel_rank(device, rank=rank, layers=1, d_model=64, d_ff=128, seed=seed)
    g = torch.Generator(device=device).manual_seed(seed * 100 + rank)
    tensors = {}
    for layer in range(layers):
        p = f"decoder.layers.{layer}.mlp.experts.local_experts.{rank}."
        for name, shape in (("w1", (d_ff, d_model)), ("w3", (d_ff, d_model)), ("w2", (d_model, d_ff))):
            tensors[p + name] = torch.randn(shape, device=device, dtype=torch.bfloat16, generator=g) * 0.02
        tensors[f"decoder.layers.{layer}.router.weight"] = torch.randn((8, d_model), device=device, dtype=torch.bfloat16, generator=g) * 0.02
    for name, t in small["tensors"].items():
        if t.device.type == "cpu":
            tensors[name] = t
    return {"tensors": tensors, "blobs": small["blobs"], "bucket_count": 1}


def gpt2_small_adam(device, seed=0, layers=12, d_model=768, d_ff=3072, vocab=50257, ctx=1024):
    """GPT-2 small (tied embeddings, 124 439 808 parameters) with Adam state, all fp32: weights
    N(0, 0.02) with LayerNorm gains 1.0, ``exp_avg`` N(0, 1e-3), ``exp_avg_sq`` its square-law
    counterpart, and one int64 ``step`` scalar (1000) per parameter: 12 bytes per parameter, 1.49 GB.
    Values are drawn on ``device`` from a generator seeded with ``seed`` alone, so every rank of a
    data-parallel job (same device type) holds the same replica."""
    g = torch.Generator(device=device).manual_seed(seed)
    shapes = [("transformer.wte.weight", (vocab, d_model)), ("transformer.wpe.weight", (ctx, d_model))]
    for i in range(layers):
        p = f"transformer.h.{i}."
        shapes += [
            (p + "ln_1.weight", (d_model,)), (p + "ln_1.bias", (d_model,)),
            (p + "attn.c_attn.weight", (d_model, 3 * d_model)), (p + "attn.c_attn.bias", (3 * d_model,)),
            (p + "attn.c_proj.weight", (d_model, d_model)), (p + "attn.c_proj.bias", (d_model,)),
            (p + "ln_2.weight", (d_model,)), (p + "ln_2.bias", (d_model,)),
            (p + "mlp.c_fc.weight", (d_model, d_ff)), (p + "mlp.c_fc.bias", (d_ff,)),
            (p + "mlp.c_proj.weight", (d_ff, d_model)), (p + "mlp.c_proj.bias", (d_model,)),
        ]
    shapes += [("transformer.ln_f.weight", (d_model,)), ("transformer.ln_f.bias", (d_model,))]
    state = {}
    for name, shape in shapes:
        w = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 0.02
        if ".ln_" in name and name.endswith("weight"):
            w.fill_(1.0)
        state["model." + name] = w
        state["optim.exp_avg." + name] = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 1e-3
        state["optim.exp_avg_sq." + name] = (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 1e-3) ** 2
        state["optim.step." + name] = torch.tensor(1000, dtype=torch.int64, device=device)
    return state
