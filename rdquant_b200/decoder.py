"""A Qwen3-architecture decoder over the fused mixed-precision linears, for whole-model
prefill / greedy-decode measurements on synthetic weights (BASELINE configs 4 and 5; the
reference's harness is benchmarks/bench_e2e.py:103-155 over a HuggingFace model).

q/k/v and gate/up are packed as one layer each (they read the same input).  In the prefill pass
everything that is not a linear layer -- embedding lookup, RMSNorm, rotary embedding, attention,
SiLU x mul, residual adds -- is plain PyTorch.  A decode step uses the kernels of csrc/rdq_glue.cu
instead, chained by programmatic dependent launch with the GEMVs: on one GPU a block is five
launches -- q+k+v GEMV with the add + RMSNorm as its activation prologue, one launch for q/k norm +
rotary + cache write + attention, o GEMV, gate+up GEMV (add + RMSNorm prologue), down GEMV (SiLU x
mul prologue); where a prologue does not apply (larger batches, several GPUs) the same steps run
as kernels of their own.  ``fused_glue=False`` runs the PyTorch operators of the prefill instead;
the embedding lookup, the FP16 lm_head and the arg-max are PyTorch in both.  A decode step has
static shapes (the KV cache is allocated for the whole run, the current position lives in a
device tensor), so it is captured once in a CUDA graph and replayed per token.

With ``world > 1`` every linear is column-parallel: each rank streams its rows and the full
activation is rebuilt on every rank -- by stores into every GPU's gather buffer from the GEMV's
epilogue (``parallel.PeerGatherMixedLinear``, the default) or by one NCCL all-gather per linear
(``parallel.ColumnParallelMixedLinear``, ``peer_gather=False``, and always for the prefill GEMM);
the glue is computed redundantly on all ranks.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from rdquant_b200.fused_gemv_pack import fuse_layers, packed_weight_bytes
from rdquant_b200.quantize import quantize_weight_packed


@dataclass
class DecoderConfig:
    layers: int = 36
    hidden: int = 2560
    ffn: int = 9728
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    vocab: int = 151936
    qk_norm: bool = True
    rope_theta: float = 1.0e6
    eps: float = 1.0e-6
    frac_fp4: float = 0.67
    frac_fp16: float = 0.01
    name: str = "qwen3-4b-shaped"


QWEN3_4B = DecoderConfig()
LLAMA3_70B = DecoderConfig(layers=80, hidden=8192, ffn=28672, q_heads=64, kv_heads=8, head_dim=128, vocab=128256,
                           qk_norm=False, rope_theta=5.0e5, eps=1.0e-5, frac_fp4=0.85, frac_fp16=0.0,
                           name="llama3-70b-shaped")


def _splits(n_out: int, cfg: DecoderConfig) -> dict:
    """Channel counts per format: the configured fractions rounded to 128 channels (layers
    narrower than three tiles: to 16 channels, like synthetic.fixed_splits)."""
    unit = 128 if n_out >= 384 else 16
    rnd = lambda v: int(round(v / unit)) * unit  # noqa: E731
    n16 = max(unit, rnd(cfg.frac_fp16 * n_out)) if cfg.frac_fp16 > 0 else 0
    n4 = min(rnd(cfg.frac_fp4 * n_out), n_out - n16)
    return {"NVFP4": n4, "FP8": n_out - n4 - n16, "FP16": n16}


def _rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, T, H, D]; cos / sin [T, D] (halves duplicated, HuggingFace convention)."""
    d = x.shape[-1] // 2
    rot = torch.cat([-x[..., d:], x[..., :d]], dim=-1)
    return x * cos[None, :, None, :] + rot * sin[None, :, None, :]


class MixedDecoder:
    """Random-init decoder; weights are generated, encoded and packed layer by layer on the GPU."""

    def __init__(self, cfg: DecoderConfig, device, max_seq: int, batch: int, seed: int = 0, rank: int = 0,
                 world: int = 1, group=None, use_pdl: bool = True, fused_glue: bool = True, peer_gather: bool = True,
                 fuse_prologue=True, fused_attention: bool = True, random_perm: bool = False) -> None:
        self.cfg, self.device, self.max_seq, self.batch = cfg, torch.device(device), max_seq, batch
        self.rank, self.world, self.group = rank, world, group
        self.use_pdl, self.fused_glue, self.fuse_prologue = use_pdl, fused_glue, fuse_prologue
        self.fused_attention = fused_attention and cfg.head_dim in (64, 128, 256)
        self.random_perm = random_perm
        self.arena = None
        if world > 1 and peer_gather:
            from rdquant_b200.parallel import PeerArena

            widest = max(cfg.q_heads * cfg.head_dim + 2 * cfg.kv_heads * cfg.head_dim, 2 * cfg.ffn, cfg.hidden)
            per_layer = 4 * ((widest // world + 256) * world * 16 * 2 + 1024)
            self.arena = PeerArena(cfg.layers * per_layer, self.device, group)
        gen = torch.Generator(device=self.device).manual_seed(seed)
        h, dh = cfg.hidden, cfg.head_dim
        nq, nkv = cfg.q_heads * dh, cfg.kv_heads * dh
        self.linear_bytes = 0       # packed weight + scale bytes of all linears (whole model)
        self.local_linear_bytes = 0  # ... of this rank's rows
        self.blocks = []
        for _ in range(cfg.layers):
            blk = {
                "qkv": self._linear([(h, nq), (h, nkv), (h, nkv)], gen, use_pdl),
                "o": self._linear([(nq, h)], gen, use_pdl),
                "gate_up": self._linear([(h, cfg.ffn), (h, cfg.ffn)], gen, use_pdl),
                "down": self._linear([(cfg.ffn, h)], gen, use_pdl),
                "ln1": torch.ones(h, dtype=torch.float16, device=self.device),
                "ln2": torch.ones(h, dtype=torch.float16, device=self.device),
                "qn": torch.ones(dh, dtype=torch.float16, device=self.device),
                "kn": torch.ones(dh, dtype=torch.float16, device=self.device),
            }
            self.blocks.append(blk)
        self.embed = (torch.randn(cfg.vocab, h, generator=gen, device=self.device, dtype=torch.float32) * 0.02).half()
        self.lm_head = self.embed  # tied, FP16 (not quantised), like the checkpoint's embed / lm_head
        self.norm = torch.ones(h, dtype=torch.float16, device=self.device)
        inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, dh, 2, device=self.device).float() / dh))
        ang = torch.arange(max_seq, device=self.device).float()[:, None] * inv_freq[None, :]
        self.cos = torch.cat([ang.cos(), ang.cos()], dim=-1).half()
        self.sin = torch.cat([ang.sin(), ang.sin()], dim=-1).half()
        self.positions = torch.arange(max_seq, device=self.device)
        self.reset(batch)

    def reset(self, batch: int) -> None:
        """(Re)allocate the KV cache and the step state for `batch` sequences; drops a captured graph."""
        cfg = self.cfg
        self.batch = batch
        self._graph = None
        for blk in self.blocks:
            blk["k"] = torch.zeros(batch, cfg.kv_heads, self.max_seq, cfg.head_dim, dtype=torch.float16, device=self.device)
            blk["v"] = torch.zeros(batch, cfg.kv_heads, self.max_seq, cfg.head_dim, dtype=torch.float16, device=self.device)
        self.pos = torch.zeros(1, dtype=torch.long, device=self.device)      # next position to write
        self.ids = torch.zeros(batch, dtype=torch.long, device=self.device)  # tokens fed to the next step
        from rdquant_b200 import rdquant_cuda

        f16 = dict(dtype=torch.float16, device=self.device)
        self._bufs = {
            "x": torch.zeros(batch, cfg.hidden, **f16), "x2": torch.zeros(batch, cfg.hidden, **f16),
            "h": torch.zeros(batch, cfg.hidden, **f16), "down": torch.zeros(batch, cfg.hidden, **f16),
            "qkv": torch.zeros(batch, (cfg.q_heads + 2 * cfg.kv_heads) * cfg.head_dim, **f16),
            "gu": torch.zeros(batch, 2 * cfg.ffn, **f16),
            "q": torch.zeros(batch, cfg.q_heads, cfg.head_dim, **f16),
            "att": torch.zeros(batch, cfg.q_heads * cfg.head_dim, **f16), "act": torch.zeros(batch, cfg.ffn, **f16),
            "scratch": rdquant_cuda.attn_decode_scratch(batch, cfg.q_heads, cfg.head_dim, self.max_seq, self.device),
            "scratch2": rdquant_cuda.rope_attn_scratch(batch, cfg.q_heads, cfg.kv_heads, cfg.head_dim, self.max_seq,
                                                       self.device),
        }

    # ---- construction
    def _permutation(self, n, sp, gen):
        """Channel order of a layer: a random assignment of the channels to the formats, grouped by
        format with the original order kept inside a group -- what the reference's allocator
        produces (rdquant/core/allocator.py:210-224).  ``random_perm=True`` shuffles all channels
        instead (the worst case for the locality of the output stores)."""
        if self.random_perm:
            return torch.randperm(n, generator=gen, device=self.device)
        shuffled = torch.randperm(n, generator=gen, device=self.device)
        parts, off = [], 0
        for fmt in ("NVFP4", "FP8", "FP16"):
            parts.append(shuffled[off:off + sp[fmt]].sort().values)
            off += sp[fmt]
        return torch.cat(parts)

    def _linear(self, shapes, gen, use_pdl):
        cfg = self.cfg
        parts = []
        for k, n in shapes:
            w = (torch.randn(n, k, generator=gen, device=self.device, dtype=torch.float32) * 0.02)
            idx = torch.randperm(n, generator=gen, device=self.device)[: n // 100]
            w[idx] *= 8
            sp = _splits(n, cfg)
            perm = self._permutation(n, sp, gen)
            parts.append((quantize_weight_packed(w.half(), perm, sp), sp))
            self.linear_bytes += packed_weight_bytes(sp, k)
            del w
        k = shapes[0][0]
        data, sp = fuse_layers(parts) if len(parts) > 1 else parts[0]
        if self.world > 1:
            from rdquant_b200.parallel import ColumnParallelMixedLinear, PeerGatherMixedLinear

            if self.arena is not None:
                mod = PeerGatherMixedLinear(data, sp, k, self.arena)
            else:
                mod = ColumnParallelMixedLinear(data, sp, k, self.device, self.rank, self.world, self.group)
            self.local_linear_bytes += mod.packed_bytes()
        else:
            from rdquant_b200.inference import FusedMixedLinear

            mod = FusedMixedLinear.from_layer_data(data, sp, k, self.device)
            self.local_linear_bytes += packed_weight_bytes(sp, k)
        mod.use_pdl = use_pdl
        return mod

    # ---- one forward pass over `t` new tokens per sequence, written at positions pos .. pos + t - 1
    def _forward(self, ids: torch.Tensor, t: int, pos0) -> torch.Tensor:
        """ids [B, t]; pos0: int (prefill) or the device tensor self.pos (graphed decode, t == 1).
        Returns the logits of the last position [B, vocab]."""
        cfg = self.cfg
        b = ids.shape[0]
        x = self.embed[ids]  # [B, t, H]
        if isinstance(pos0, int):
            cos, sin = self.cos[pos0:pos0 + t], self.sin[pos0:pos0 + t]
            idx = self.positions[pos0:pos0 + t]
            mask = (self.positions[None, :] <= idx[:, None])[None, None]  # [1, 1, t, S]
        else:
            cos, sin = self.cos.index_select(0, pos0), self.sin.index_select(0, pos0)
            idx = pos0
            mask = (self.positions <= pos0)[None, None, None, :]  # [1, 1, 1, S]
        nq, nkv, dh = cfg.q_heads, cfg.kv_heads, cfg.head_dim
        for blk in self.blocks:
            hcur = _rms(x, blk["ln1"], cfg.eps)
            qkv = blk["qkv"](hcur)
            q = qkv[..., : nq * dh].reshape(b, t, nq, dh)
            k = qkv[..., nq * dh:(nq + nkv) * dh].reshape(b, t, nkv, dh)
            v = qkv[..., (nq + nkv) * dh:].reshape(b, t, nkv, dh)
            if cfg.qk_norm:
                q, k = _rms(q, blk["qn"], cfg.eps), _rms(k, blk["kn"], cfg.eps)
            q, k = _rope(q, cos, sin), _rope(k, cos, sin)
            blk["k"].index_copy_(2, idx, k.transpose(1, 2))
            blk["v"].index_copy_(2, idx, v.transpose(1, 2))
            att = F.scaled_dot_product_attention(q.transpose(1, 2), blk["k"], blk["v"], attn_mask=mask, enable_gqa=True)
            x = x + blk["o"](att.transpose(1, 2).reshape(b, t, nq * dh))
            hcur = _rms(x, blk["ln2"], cfg.eps)
            gu = blk["gate_up"](hcur)
            x = x + blk["down"](F.silu(gu[..., : cfg.ffn]) * gu[..., cfg.ffn:])
        last = _rms(x[:, -1], self.norm, cfg.eps)
        return last @ self.lm_head.T

    @torch.no_grad()
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """Run the prompt [B, T] (GEMM path), fill the KV cache, return the first generated ids."""
        t = ids.shape[1]
        logits = self._forward(ids, t, 0)
        self.pos.fill_(t)
        self.ids.copy_(logits.argmax(-1))
        return self.ids.clone()

    def _forward_fused(self) -> torch.Tensor:
        """One decode step (one token per sequence) with the glue kernels of rdq_glue.cu between
        the linears instead of framework operators.  On one GPU the norms and the MLP activation
        run inside the GEMV that consumes them (activation prologue) where the batch allows:
        6 launches per block instead of 9."""
        from rdquant_b200 import _lib, rdquant_cuda as rc

        cfg, st = self.cfg, self._bufs
        flags = _lib.RDQ_GEMV_PDL if self.use_pdl else 0
        b = self.batch
        fuse = self.world == 1 and bool(self.fuse_prologue) and b <= rc.MAX_GEMV_M
        fuse_norm = fuse and self.fuse_prologue in (True, "norm") and rc.gemv_stages_x(b, cfg.hidden)
        fuse_act = fuse and self.fuse_prologue in (True, "act") and rc.gemv_stages_x(b, cfg.ffn)
        cur, other, hbuf = st["x"], st["x2"], st["h"]
        torch.index_select(self.embed, 0, self.ids, out=cur)
        delta = None
        scale = cfg.head_dim ** -0.5

        def norm_linear(mod, w, out):
            # residual += delta; out = rmsnorm(residual) @ W.T
            nonlocal cur, other
            if fuse_norm:
                rc.mixed_gemv_norm(cur, delta, w, cfg.eps, mod._fd(), residual_out=other, flags=flags, out=out)
                cur, other = other, cur
                return out
            rc.add_rmsnorm(cur, delta, w, hbuf, cfg.eps, flags)
            return mod(hbuf)

        for blk in self.blocks:
            qkv = norm_linear(blk["qkv"], blk["ln1"], st["qkv"])
            if self.fused_attention:
                rc.rope_attn_decode(qkv, blk["qn"] if cfg.qk_norm else None, blk["kn"] if cfg.qk_norm else None, self.cos,
                                    self.sin, self.pos, blk["k"], blk["v"], st["scratch2"], st["att"], cfg.q_heads, scale,
                                    cfg.eps, flags)
            else:
                rc.qk_rope_cache(qkv, blk["qn"] if cfg.qk_norm else None, blk["kn"] if cfg.qk_norm else None, self.cos,
                                 self.sin, self.pos, st["q"], blk["k"], blk["v"], cfg.eps, flags)
                rc.attn_decode(st["q"], blk["k"], blk["v"], self.pos, st["scratch"], st["att"], scale, flags)
            delta = blk["o"](st["att"])
            gu = norm_linear(blk["gate_up"], blk["ln2"], st["gu"])
            if fuse_act:
                delta = rc.mixed_gemv_silu(gu, blk["down"]._fd(), flags=flags, out=st["down"])
            else:
                rc.silu_mul(gu, st["act"], flags)
                delta = blk["down"](st["act"])
        rc.add_rmsnorm(cur, delta, self.norm, hbuf, cfg.eps, flags)
        return hbuf @ self.lm_head.T

    def _step(self) -> None:
        if self.fused_glue:
            logits = self._forward_fused()
        else:
            logits = self._forward(self.ids[:, None], 1, self.pos)
        self.ids.copy_(logits.argmax(-1))
        self.pos.add_(1)

    @torch.no_grad()
    def capture_decode(self) -> None:
        """Capture one decode step (static shapes) into a CUDA graph; replay with ``decode_step``."""
        pos_saved, ids_saved = self.pos.clone(), self.ids.clone()
        stream = torch.cuda.Stream(self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            for _ in range(2):  # warm-up outside capture: lazy initialisation, buffer allocation
                self._step()
            stream.synchronize()
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph, stream=stream):
                self._step()
        torch.cuda.current_stream(self.device).wait_stream(stream)
        self.pos.copy_(pos_saved)
        self.ids.copy_(ids_saved)

    def release_graph(self) -> None:
        """Drop the captured step (before a process group whose collectives it holds goes away)."""
        self._graph = None

    @torch.no_grad()
    def decode_step(self) -> None:
        if self._graph is None:
            self._step()
        else:
            self._graph.replay()
