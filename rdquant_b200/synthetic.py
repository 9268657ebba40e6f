"""Seeded synthetic layers with the shapes and value distributions of the benchmark
configurations: weights ~ N(0, 0.02) in float16 with 1 % of output channels scaled x8,
activations ~ N(0, 1), fixed 67/32/1 NVFP4/FP8/FP16 channel split rounded to 128
channels, random channel permutation."""
from __future__ import annotations

import torch

from rdquant_b200.quantize import QuantizedWeight, quantize_weight

# (K, N) of the seven linears of one Qwen3-4B decoder block
QWEN3_4B_BLOCK = {
    "q_proj": (2560, 4096),
    "k_proj": (2560, 1024),
    "v_proj": (2560, 1024),
    "o_proj": (4096, 2560),
    "gate_proj": (2560, 9728),
    "up_proj": (2560, 9728),
    "down_proj": (9728, 2560),
}


def _round128(v: float) -> int:
    return int(round(v / 128.0)) * 128


def fixed_splits(n_out: int, frac_fp4: float = 0.67, frac_fp16: float = 0.01) -> dict:
    """``n16 = max(128, round128(frac_fp16 N))``, ``n4 = round128(frac_fp4 N)``, rest FP8."""
    if n_out < 384:
        n4 = (n_out // 2) // 16 * 16
        n16 = 16 if n_out >= 48 else 0
        return {"NVFP4": n4, "FP8": n_out - n4 - n16, "FP16": n16}
    n16 = max(128, _round128(frac_fp16 * n_out)) if frac_fp16 > 0 else 0
    n4 = _round128(frac_fp4 * n_out)
    return {"NVFP4": n4, "FP8": n_out - n4 - n16, "FP16": n16}


def synthetic_weight(n_out: int, n_in: int, gen: torch.Generator) -> torch.Tensor:
    w = (torch.randn(n_out, n_in, generator=gen) * 0.02).half()
    idx = torch.randperm(n_out, generator=gen)[: max(n_out // 100, 0)]
    w[idx] *= 8
    return w


def synthetic_layer(n_in: int, n_out: int, seed: int = 0, splits: dict | None = None,
                    random_perm: bool = True) -> tuple[QuantizedWeight, torch.Tensor]:
    """(quantised weight on CPU, the float16 source weight)."""
    gen = torch.Generator().manual_seed(seed)
    w = synthetic_weight(n_out, n_in, gen)
    splits = splits or fixed_splits(n_out)
    perm = torch.randperm(n_out, generator=gen) if random_perm else torch.arange(n_out)
    return quantize_weight(w.float(), perm, splits), w


def random_packed_layer(n4: int, n8: int, n16: int, k: int, seed: int = 0, device="cpu",
                        per_channel_fp8: bool = True) -> dict:
    """Random *bytes* in the checkpoint layout (every code and scale pattern occurs,
    NaN patterns excluded), the way the reference's kernel tests build inputs
    (tests/test_fused_inference.py:45-59)."""
    gen = torch.Generator().manual_seed(seed)
    n = n4 + n8 + n16
    data = {"inv_permutation": torch.randperm(n, generator=gen).to(torch.int32)}

    def rand_e4m3(shape, positive=False):
        b = torch.randint(0, 256, shape, generator=gen, dtype=torch.int32)
        b = torch.where((b & 0x7F) == 0x7F, b - 1, b)  # 0x7f / 0xff are NaN
        if positive:
            b = b & 0x7F
        return b.to(torch.uint8)

    if n4:
        data["weight_nvfp4"] = torch.randint(0, 256, (n4, k // 2), generator=gen, dtype=torch.int32).to(torch.uint8)
        # block scales at most 16 so that sums of hundreds of products stay inside float16
        sc = rand_e4m3((n4, k // 16), positive=True)
        data["weight_nvfp4_scale"] = torch.minimum(sc, torch.tensor(0x58, dtype=torch.uint8))
        data["nvfp4_global_scale"] = torch.ones(1)
    if n8:
        w8 = rand_e4m3((n8, k))
        data["weight_fp8"] = w8
        if per_channel_fp8:
            data["weight_fp8_scale"] = (torch.rand(n8, generator=gen) * 0.01 + 1e-3).float()
        else:
            data["weight_fp8_scale"] = torch.full((n8,), 0.004, dtype=torch.float32)
    if n16:
        data["weight_fp16"] = (torch.randn(n16, k, generator=gen) * 0.05).to(torch.bfloat16)
    return {kk: v.to(device) for kk, v in data.items()}
