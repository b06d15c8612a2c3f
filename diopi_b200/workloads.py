"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configs.

No dataset or benchmark suite stands behind this path; every input is generated. Index tensors are
drawn with a CPU generator (identical on every machine and rank), float data with a generator on the
target device. Used by bench.py, the tests and the smoke check.

  decode("cfg1")  B4  H8  D64  fp32, lens in [16,128], pool = sum(lens)+64      (CPU-runnable case)
  decode("cfg2")  B64 H32 D128 fp16, lens in [512,4096], pool = 64*4096         (LLaMA-7B decode)
  decode("cfg5")  B128 H64 D128 fp16, lens in [1024,8192], pool = sum(lens)+128 (64-head decode)
  prenorm()       8192 x 4096 bf16 RMSNorm + rotary on [8192,32,128]
  prefill()       B8 H32 D128 fp16, lens in [1024,8192], packed ragged
  penalty()       fp32 logits [128,32000], up to 512 distinct prior ids per request
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

DECODE_CONFIGS = {
    # name: (batch, heads, head_dim, dtype, len_lo, len_hi, pool rule, kv std, seed)
    "cfg1": dict(B=4, H=8, D=64, dtype=torch.float32, lo=16, hi=128, pool="sum+64", std=1.0, seed=1001),
    "cfg2": dict(B=64, H=32, D=128, dtype=torch.float16, lo=512, hi=4096, pool="B*hi", std=0.5, seed=1002),
    # a quarter of cfg2 (same rows, 16 requests): small enough for a multi-pass profiler capture, still >> L2
    "cfg2s": dict(B=16, H=32, D=128, dtype=torch.float16, lo=512, hi=4096, pool="B*hi", std=0.5, seed=1012),
    # small enough for its K/V rows (67 MB) to stay in the 126 MB L2 between steps: the L2-warm variant of the step
    "cfg2w": dict(B=8, H=32, D=128, dtype=torch.float16, lo=512, hi=512, pool="sum+64", std=0.5, seed=1022),
    "cfg5": dict(B=128, H=64, D=128, dtype=torch.float16, lo=1024, hi=8192, pool="sum+128", std=0.5, seed=1005),
}


@dataclass
class DecodeWorkload:
    name: str
    q: torch.Tensor            # [B, Hs, D]
    k_pool: torch.Tensor       # [slots, Hs, D]
    v_pool: torch.Tensor
    k_new: torch.Tensor        # [B, Hs, D] this step's new K rows
    v_new: torch.Tensor
    dest_loc: torch.Tensor     # [B] int32: slot of each request's newest token
    b_loc: torch.Tensor        # [B, max_len] int32, right-aligned
    b_start_loc: torch.Tensor  # [B] int32, exclusive prefix sum of lens
    b_seq_len: torch.Tensor    # [B] int32
    max_input_len: int
    sum_len: int
    heads_total: int
    head_range: tuple = (0, 0)
    meta: dict = field(default_factory=dict)

    @property
    def elem(self) -> int:
        return self.q.element_size()

    def fused_bytes(self) -> int:
        """Algorithmic bytes of one fused decode step on this shard:
        K and V rows once, q and out once, the slot table and the two per-request index vectors."""
        B, H, D = self.q.shape
        return 2 * self.sum_len * H * D * self.elem + 2 * B * H * D * self.elem + self.sum_len * 4 + 2 * B * 4

    def copy_bytes(self) -> int:
        """Algorithmic bytes of the two DestIndexCopyKV calls of the step."""
        B, H, D = self.q.shape
        return 2 * (2 * B * H * D * self.elem + B * 4)


def decode_indices(name: str, seed: int | None = None):
    """Lengths, slot table and prefix sums of a decode config (CPU tensors, deterministic)."""
    c = DECODE_CONFIGS[name]
    g = torch.Generator().manual_seed(c["seed"] if seed is None else seed)
    B = c["B"]
    lens = torch.randint(c["lo"], c["hi"] + 1, (B,), generator=g)
    total = int(lens.sum())
    slots = {"sum+64": total + 64, "sum+128": total + 128, "B*hi": B * c["hi"]}[c["pool"]]
    perm = torch.randperm(slots, generator=g)
    max_len = int(lens.max())
    b_loc = torch.zeros(B, max_len, dtype=torch.int32)
    start = torch.zeros(B, dtype=torch.int32)
    acc = 0
    for i in range(B):
        L = int(lens[i])
        b_loc[i, max_len - L:] = perm[acc:acc + L].to(torch.int32)
        start[i] = acc
        acc += L
    return dict(lens=lens.to(torch.int32), b_loc=b_loc, b_start_loc=start, max_len=max_len, total=total, slots=slots)


def decode(name: str, device="cuda", head_range: tuple | None = None, float_seed: int | None = None) -> DecodeWorkload:
    """Builds a decode workload; head_range=(h0,h1) builds only that head shard of the pool."""
    c = DECODE_CONFIGS[name]
    idx = decode_indices(name)
    h0, h1 = head_range if head_range is not None else (0, c["H"])
    Hs = h1 - h0
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed((c["seed"] if float_seed is None else float_seed) * 7919 + h0)
    dt, D, B = c["dtype"], c["D"], c["B"]

    def randn(*shape, std=1.0):
        # drawn in fp32 chunks to bound the temporary, then cast
        out = torch.empty(*shape, dtype=dt, device=dev)
        flat = out.view(-1)
        step = 1 << 26
        for s in range(0, flat.numel(), step):
            n = min(step, flat.numel() - s)
            flat[s:s + n] = (torch.randn(n, generator=g, device=dev, dtype=torch.float32) * std).to(dt)
        return out

    k_pool = randn(idx["slots"], Hs, D, std=c["std"])
    v_pool = randn(idx["slots"], Hs, D, std=c["std"])
    q = randn(B, Hs, D)
    k_new = randn(B, Hs, D, std=c["std"])
    v_new = randn(B, Hs, D, std=c["std"])
    b_loc = idx["b_loc"].to(dev)
    return DecodeWorkload(
        name=name, q=q, k_pool=k_pool, v_pool=v_pool, k_new=k_new, v_new=v_new,
        dest_loc=b_loc[:, idx["max_len"] - 1].contiguous(), b_loc=b_loc,
        b_start_loc=idx["b_start_loc"].to(dev), b_seq_len=idx["lens"].to(dev),
        max_input_len=idx["max_len"], sum_len=idx["total"], heads_total=c["H"], head_range=(h0, h1),
        meta=dict(seed=c["seed"], slots=idx["slots"], dtype=str(dt).replace("torch.", "")),
    )


def shard_heads(heads: int, world: int, rank: int) -> tuple:
    """Contiguous head range of `rank` when `heads` are split as evenly as possible over `world`."""
    base, extra = divmod(heads, world)
    h0 = rank * base + min(rank, extra)
    return h0, h0 + base + (1 if rank < extra else 0)


def prenorm(device="cuda", tokens=8192, hidden=4096, heads=32, dtype=torch.bfloat16, seed=1003):
    """cfg3: x ~ N(0,1), weight ~ N(1, 0.1), cos/sin tables from theta 10000 at random positions."""
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    gc = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, hidden, generator=g, device=dev, dtype=torch.float32).to(dtype)
    w = (1 + 0.1 * torch.randn(hidden, generator=g, device=dev, dtype=torch.float32)).to(dtype)
    hd = hidden // heads
    pos = torch.randint(0, 4096, (tokens,), generator=gc).to(dev).float()
    inv_freq = 10000.0 ** (-torch.arange(0, hd, 2, device=dev, dtype=torch.float32) / hd)
    ang = pos[:, None] * inv_freq[None, :]
    cos = ang.cos().to(dtype).view(tokens, 1, hd // 2)
    sin = ang.sin().to(dtype).view(tokens, 1, hd // 2)
    k_in = torch.randn(tokens, hidden, generator=g, device=dev, dtype=torch.float32).to(dtype)
    return dict(x=x, weight=w, eps=1e-6, cos=cos, sin=sin, k_in=k_in, heads=heads, head_dim=hd)


def prefill(device="cuda", B=8, H=32, D=128, lo=1024, hi=8192, dtype=torch.float16, seed=1004):
    """cfg4: packed ragged q/k/v ~ N(0,1)/sqrt(D)."""
    dev = torch.device(device)
    gc = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (B,), generator=gc)
    total = int(lens.sum())
    start = torch.cat([torch.zeros(1, dtype=torch.int64), lens.cumsum(0)[:-1]])
    g = torch.Generator(device=dev).manual_seed(seed)
    mk = lambda: (torch.randn(total, H, D, generator=g, device=dev, dtype=torch.float32) / math.sqrt(D)).to(dtype)
    flops = int(sum(H * 4 * D * int(L) * (int(L) + 1) // 2 for L in lens))
    return dict(q=mk(), k=mk(), v=mk(), b_start_loc=start.to(torch.int32).to(dev), b_seq_len=lens.to(torch.int32).to(dev),
                max_input_len=int(lens.max()), lens=lens, flops=flops)


def penalty(device="cuda", B=128, V=32000, max_ids=512, seed=1005, dtype=torch.float32):
    """cfg5 sampling penalty: logits ~ N(0,2), penalties ~ U[0,1), distinct ids per request, counts in [1,8]."""
    dev = torch.device(device)
    gc = torch.Generator().manual_seed(seed)
    n = torch.randint(1, max_ids + 1, (B,), generator=gc)
    ids = torch.cat([torch.randperm(V, generator=gc)[: int(x)] for x in n]).to(torch.int32)
    counts = torch.randint(1, 9, (int(n.sum()),), generator=gc).to(torch.int32)
    cum = torch.cat([torch.zeros(1, dtype=torch.int64), n.cumsum(0)]).to(torch.int32)
    logits = (torch.randn(B, V, generator=gc) * 2.0).to(dtype)
    pres = torch.rand(B, generator=gc).to(dtype)
    freq = torch.rand(B, generator=gc).to(dtype)
    return dict(logits=logits.to(dev), presence=pres.to(dev), frequency=freq.to(dev), ids=ids.to(dev), counts=counts.to(dev),
                cum=cum.to(dev), max_len=int(n.max()))
