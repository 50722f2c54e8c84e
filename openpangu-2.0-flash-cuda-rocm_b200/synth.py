"""Seeded synthetic inputs with the shapes and value distributions of the MoE workloads.

No checkpoint of the model is available to this build, so every measurement and
parity case runs on synthetic tensors: activations BF16 ~N(0,1); router weight
BF16 [256,2560] ~N(0,0.02); correction bias FP32 ~N(0,0.01), zero, or fitted so
that expert popularity follows a capped Zipf law; expert weights drawn
~N(0,0.02), rounded to BF16 and quantised to NVFP4 by the library's
implementation of the offline quantiser's arithmetic (cuda/nvfp4_pack.cu:141-176,
255-256).  Each layer has its own seed.  Tensors are produced on the GPU with
torch's Philox generator, so a (seed, layer) pair names the same bytes on every
B200 run; nothing here is timed.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from . import (EXPERTS, HIDDEN, INTERMEDIATE, TOP_K, ExpertBank, nvfp4_pack_weight, nvfp4_pack_weight_batch,
               nvfp4_swizzle_scales, nvfp4_swizzled_scale_bytes)

MATRIX_BYTES = INTERMEDIATE * HIDDEN // 2      # gate, up and down all pack to 1,310,720 bytes
SCALE_BYTES = INTERMEDIATE * HIDDEN // 16      # 163,840


def _generator(seed: int, layer: int, stream: int) -> torch.Generator:
    g = torch.Generator(device="cuda")
    g.manual_seed((seed * 1_000_003 + layer * 7919 + stream) & 0x7FFFFFFFFFFFFFFF)
    return g


@dataclass
class RawLayer:
    """Reference-format tensors of one layer (what the reference keeps resident, src/resident.cpp)."""

    packed: torch.Tensor            # uint8 [(E+1)*3, MATRIX_BYTES]      entry = expert*3 + kind
    scales_linear: torch.Tensor     # uint8 [(E+1)*3, SCALE_BYTES]
    scales_swizzled: torch.Tensor   # uint8 [(E+1)*3, SCALE_BYTES]       128x4 tiled
    alpha: torch.Tensor             # float32 [(E+1)*3]                  weight_scale_2

    def entries(self):
        n = self.packed.shape[0]
        return [(self.packed[i], self.scales_swizzled[i], self.alpha[i:i + 1]) for i in range(n)]


def make_raw_layer(seed: int, layer: int, experts: int = EXPERTS, hidden: int = HIDDEN,
                   intermediate: int = INTERMEDIATE, std: float = 0.02) -> RawLayer:
    entries = (experts + 1) * 3
    mbytes = intermediate * hidden // 2
    sbytes = intermediate * hidden // 16
    packed = torch.empty((entries, mbytes), dtype=torch.uint8, device="cuda")
    linear = torch.empty((entries, sbytes), dtype=torch.uint8, device="cuda")
    swizzled = torch.empty((entries, sbytes), dtype=torch.uint8, device="cuda")
    alpha = torch.empty(entries, dtype=torch.float32, device="cuda")
    g = _generator(seed, layer, 1)
    scratch = torch.empty(intermediate * hidden, dtype=torch.float32, device="cuda")
    for i in range(entries):
        kind = i % 3
        rows, cols = (intermediate, hidden) if kind < 2 else (hidden, intermediate)
        scratch.normal_(0.0, std, generator=g)
        w = scratch.to(torch.bfloat16)
        nvfp4_pack_weight(w, packed[i], linear[i], alpha[i:i + 1])
        assert nvfp4_swizzled_scale_bytes(rows, cols // 16) == sbytes
        nvfp4_swizzle_scales(linear[i], swizzled[i], rows, cols // 16)
    return RawLayer(packed, linear, swizzled, alpha)


def make_raw_layer_batched(seed: int, layer: int, experts: int = EXPERTS, hidden: int = HIDDEN,
                           intermediate: int = INTERMEDIATE, std: float = 0.02) -> RawLayer:
    """The same distributions as make_raw_layer in a dozen launches instead of several thousand: all
    matrices of the layer are drawn by one call of the generator (so the bytes differ from
    make_raw_layer's for the same seed), quantised by the batched weight quantiser, and their scales
    tiled per matrix shape (equally shaped matrices stored back to back tile like one tall matrix,
    because every matrix has a multiple of 128 rows).  Used where set-up time matters: the smoke test
    and the benchmark's 44 layers."""
    n = experts + 1
    elements = intermediate * hidden
    g = _generator(seed, layer, 4)
    w = torch.empty((3 * n, elements), dtype=torch.bfloat16, device="cuda").normal_(0.0, std, generator=g)   # [kind][entry]
    packed = torch.empty((3 * n, elements // 2), dtype=torch.uint8, device="cuda")
    linear = torch.empty((3 * n, elements // 16), dtype=torch.uint8, device="cuda")
    swizzled = torch.empty_like(linear)
    alpha = torch.empty(3 * n, dtype=torch.float32, device="cuda")
    nvfp4_pack_weight_batch(w, packed, linear, alpha)
    del w
    nvfp4_swizzle_scales(linear[:2 * n], swizzled[:2 * n], 2 * n * intermediate, hidden // 16)
    nvfp4_swizzle_scales(linear[2 * n:], swizzled[2 * n:], n * hidden, intermediate // 16)

    def by_entry(t):            # [kind][entry] -> [entry][kind], the reference's bank order
        return t.view(3, n, -1).transpose(0, 1).contiguous().view(3 * n, -1)

    return RawLayer(by_entry(packed), by_entry(linear), by_entry(swizzled), by_entry(alpha).view(-1))


@dataclass
class Layer:
    router_weight: torch.Tensor     # bf16 [256, hidden]
    bias: torch.Tensor              # f32 [256]
    bank: ExpertBank
    raw: Optional[RawLayer] = None
    info: dict = field(default_factory=dict)


def make_router(seed: int, layer: int, hidden: int = HIDDEN, bias_std: float = 0.01):
    g = _generator(seed, layer, 2)
    w = torch.empty((EXPERTS, hidden), dtype=torch.float32, device="cuda").normal_(0.0, 0.02, generator=g)
    b = torch.empty(EXPERTS, dtype=torch.float32, device="cuda").normal_(0.0, bias_std, generator=g)
    if bias_std == 0.0:
        b.zero_()
    return w.to(torch.bfloat16), b


def make_activations(seed: int, layer: int, rows: int, hidden: int = HIDDEN) -> torch.Tensor:
    g = _generator(seed, layer, 3)
    return torch.empty((rows, hidden), dtype=torch.float32, device="cuda").normal_(0.0, 1.0, generator=g).to(
        torch.bfloat16)


def host_router_inputs(seed: int, layer: int, rows: int, bias_std: float = 0.01, hidden: int = HIDDEN, stream: int = 0):
    """Router weight, correction bias and token rows of one layer drawn on the HOST (numpy), as BF16 / FP32
    torch CPU tensors: the one generator a GPU run and a CPU run of the same workload both take their routing
    inputs from, so that both route the same tokens to the same experts.  `stream` separates the token rows of
    different ranks; router weight and bias depend on (seed, layer) only."""
    import numpy as np

    rng = np.random.default_rng([seed, layer])
    router = torch.from_numpy((rng.standard_normal((EXPERTS, hidden), dtype=np.float32) * np.float32(0.02))).to(torch.bfloat16)
    bias = torch.from_numpy((rng.standard_normal(EXPERTS, dtype=np.float32) * np.float32(bias_std)))
    rng_x = np.random.default_rng([seed, layer, 7, stream])
    x = torch.from_numpy(rng_x.standard_normal((rows, hidden), dtype=np.float32)).to(torch.bfloat16)
    return router, bias, x


def zipf_target(alpha: float, seed: int, experts: int = EXPERTS, top_k: int = TOP_K) -> torch.Tensor:
    """Share of assignments per expert: min(1/top_k, c * rank^-alpha), c solved so shares sum to 1,
    ranks assigned by a seeded permutation of the expert ids.  (An expert is chosen at most once per
    token, so no share can exceed 1/top_k; a pure Zipf(1.2) head would.)"""
    ranks = torch.arange(1, experts + 1, dtype=torch.float64)
    base = ranks.pow(-alpha)
    lo, hi = 0.0, 1e6
    for _ in range(200):
        c = 0.5 * (lo + hi)
        total = torch.clamp(c * base, max=1.0 / top_k).sum().item()
        lo, hi = (c, hi) if total < 1.0 else (lo, c)
    share = torch.clamp(0.5 * (lo + hi) * base, max=1.0 / top_k)
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    perm = torch.randperm(experts, generator=g)
    out = torch.empty(experts, dtype=torch.float64)
    out[perm] = share
    return out.to(torch.float32)


def fit_zipf_bias(router_weight: torch.Tensor, alpha: float, seed: int, sample_rows: int = 8192,
                  iterations: int = 60) -> tuple:
    """Fixed-iteration fit of the correction bias so top-8 popularity follows zipf_target().
    Returns (bias, achieved share).  Scores use a plain FP32 matmul; this shapes the workload,
    it is not the router under test."""
    target = zipf_target(alpha, seed).cuda()
    x = make_activations(seed, 10_000, sample_rows, router_weight.shape[1]).float()
    score = torch.sigmoid(x @ router_weight.float().t())
    bias = torch.zeros(EXPERTS, dtype=torch.float32, device="cuda")
    achieved = None
    for it in range(iterations):
        top = torch.topk(score + bias, TOP_K, dim=1).indices
        achieved = torch.bincount(top.reshape(-1), minlength=EXPERTS).float() / top.numel()
        step = 0.05 if it < 40 else 0.02
        bias += step * (torch.log(target + 1e-6) - torch.log(achieved + 1e-6))
        bias -= bias.mean()
    return bias, achieved


def make_layer(seed: int, layer: int, bias_mode: str = "normal", zipf_alpha: float = 1.2,
               keep_raw: bool = False, batched: bool = False) -> Layer:
    """bias_mode: 'normal' (~N(0,0.01)), 'zero', or 'zipf' (fitted, see fit_zipf_bias).
    batched: draw and quantise the layer with make_raw_layer_batched (other bytes, same distributions)."""
    router_weight, bias = make_router(seed, layer, bias_std=0.0 if bias_mode == "zero" else 0.01)
    info = {}
    if bias_mode == "zipf":
        bias, achieved = fit_zipf_bias(router_weight, zipf_alpha, seed + layer)
        info["zipf_share_max"] = float(achieved.max())
    raw = make_raw_layer_batched(seed, layer) if batched else make_raw_layer(seed, layer)
    bank = ExpertBank(raw.entries())
    torch.cuda.synchronize()
    return Layer(router_weight, bias.contiguous(), bank, raw if keep_raw else None, info)
