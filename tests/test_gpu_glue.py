"""Decode-step glue kernels (csrc/rdq_glue.cu) through the C ABI against plain PyTorch FP32
restatements of the same formulas."""
import pytest
import torch
import torch.nn.functional as F

from rdquant_b200 import _lib, rdquant_cuda as rc

pytestmark = pytest.mark.gpu


def _close(a, b, tol=2e-3):
    err = (a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6)
    assert float(err) < tol, float(err)


@pytest.mark.parametrize("b,h", [(1, 2560), (8, 2560), (3, 8192), (2, 256)])
@pytest.mark.parametrize("with_delta", [False, True])
def test_add_rmsnorm(b, h, with_delta):
    g = torch.Generator().manual_seed(b + h)
    x = torch.randn(b, h, generator=g).half().cuda()
    d = torch.randn(b, h, generator=g).half().cuda() if with_delta else None
    w = (1 + 0.1 * torch.randn(h, generator=g)).half().cuda()
    out = torch.empty_like(x)
    x_ref = (x + d) if with_delta else x.clone()
    xf = x_ref.float()
    ref = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).half() * w
    rc.add_rmsnorm(x, d, w, out, 1e-6, _lib.RDQ_GEMV_PDL)
    assert torch.equal(x, x_ref)
    _close(out, ref)


@pytest.mark.parametrize("b,nq,nkv,dh,norm", [(1, 32, 8, 128, True), (4, 8, 2, 64, True), (2, 64, 8, 128, False)])
def test_qk_rope_cache_and_attention(b, nq, nkv, dh, norm):
    s, pos_v = 96, 37
    g = torch.Generator().manual_seed(nq + dh)
    qkv = torch.randn(b, (nq + 2 * nkv) * dh, generator=g).half().cuda()
    qn = (1 + 0.1 * torch.randn(dh, generator=g)).half().cuda() if norm else None
    kn = (1 + 0.1 * torch.randn(dh, generator=g)).half().cuda() if norm else None
    inv_freq = 1.0 / (1e6 ** (torch.arange(0, dh, 2).float() / dh))
    ang = torch.arange(s).float()[:, None] * inv_freq[None, :]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1).half().cuda(), torch.cat([ang.sin(), ang.sin()], -1).half().cuda()
    k_cache = (torch.randn(b, nkv, s, dh, generator=g) * 0.5).half().cuda()
    v_cache = torch.randn(b, nkv, s, dh, generator=g).half().cuda()
    k0, v0 = k_cache.clone(), v_cache.clone()
    pos = torch.tensor([pos_v], dtype=torch.long, device="cuda")
    q_out = torch.empty(b, nq, dh, dtype=torch.float16, device="cuda")
    rc.qk_rope_cache(qkv, qn, kn, cos, sin, pos, q_out, k_cache, v_cache, 1e-6, _lib.RDQ_GEMV_PDL)

    def rms(x, w):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)).half() * w

    def rope(x):
        xf, c, sn = x.float(), cos[pos_v].float(), sin[pos_v].float()
        rot = torch.cat([-xf[..., dh // 2:], xf[..., : dh // 2]], -1)
        return (xf * c + rot * sn).half()

    q = qkv[:, : nq * dh].reshape(b, nq, dh)
    k = qkv[:, nq * dh:(nq + nkv) * dh].reshape(b, nkv, dh)
    v = qkv[:, (nq + nkv) * dh:].reshape(b, nkv, dh)
    if norm:
        q, k = rms(q, qn), rms(k, kn)
    _close(q_out, rope(q))
    _close(k_cache[:, :, pos_v], rope(k))
    assert torch.equal(v_cache[:, :, pos_v], v)
    keep = torch.ones(s, dtype=torch.bool)
    keep[pos_v] = False
    assert torch.equal(k_cache[:, :, keep], k0[:, :, keep]) and torch.equal(v_cache[:, :, keep], v0[:, :, keep])

    scratch = rc.attn_decode_scratch(b, nq, dh, s, "cuda")
    out = torch.empty(b, nq * dh, dtype=torch.float16, device="cuda")
    rc.attn_decode(q_out, k_cache, v_cache, pos, scratch, out, dh ** -0.5, _lib.RDQ_GEMV_PDL)
    mask = (torch.arange(s, device="cuda") <= pos_v)[None, None, None, :]
    ref = F.scaled_dot_product_attention(q_out[:, :, None, :].float(), k_cache.float(), v_cache.float(), attn_mask=mask,
                                         enable_gqa=True)
    _close(out, ref.reshape(b, nq * dh))


@pytest.mark.parametrize("b,f", [(1, 9728), (8, 9728), (3, 512)])
def test_silu_mul(b, f):
    g = torch.Generator().manual_seed(f)
    gu = (torch.randn(b, 2 * f, generator=g) * 2).half().cuda()
    out = torch.empty(b, f, dtype=torch.float16, device="cuda")
    rc.silu_mul(gu, out, _lib.RDQ_GEMV_PDL)
    _close(out, F.silu(gu[:, :f].float()) * gu[:, f:].float())


def test_bad_shapes_raise():
    x = torch.zeros(2, 12, dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError):
        rc.add_rmsnorm(x, None, torch.ones(12, dtype=torch.float16, device="cuda"), torch.empty_like(x), 1e-6)
    with pytest.raises(RuntimeError):
        rc.silu_mul(torch.zeros(2, 30, dtype=torch.float16, device="cuda"), torch.zeros(2, 16, dtype=torch.float16, device="cuda"))


@pytest.mark.parametrize("b,nq,nkv,dh,norm,s,pos_v", [
    (1, 32, 8, 128, True, 776, 520),    # the measurement decoder's geometry: 7 splits, 6 used
    (1, 32, 8, 128, True, 776, 0),      # first token: one row, one split used
    (1, 32, 8, 128, True, 776, 775),    # last row of the cache
    (4, 8, 2, 64, True, 96, 37),        # one split, head_dim 64
    (2, 64, 8, 128, False, 1500, 1333),  # 8 query heads per KV head (two per warp), several tiles per split
    (1, 4, 4, 256, True, 5000, 4100),   # head_dim 256, one query head per KV head, 32 splits, 5 tiles per split
    (3, 6, 2, 128, False, 200, 64),     # 3 query heads per KV head; the new row opens a 32-row block
])
def test_rope_attn_decode_single_launch(b, nq, nkv, dh, norm, s, pos_v):
    """The one-launch rotary + cache write + attention gives the cache rows of rdq_qk_rope_cache
    bit for bit and the output of rdq_attn_decode (another summation order: FP32 tolerance)."""
    g = torch.Generator().manual_seed(nq + dh + pos_v)
    qkv = torch.randn(b, (nq + 2 * nkv) * dh, generator=g).half().cuda()
    qn = (1 + 0.1 * torch.randn(dh, generator=g)).half().cuda() if norm else None
    kn = (1 + 0.1 * torch.randn(dh, generator=g)).half().cuda() if norm else None
    inv_freq = 1.0 / (1e6 ** (torch.arange(0, dh, 2).float() / dh))
    ang = torch.arange(s).float()[:, None] * inv_freq[None, :]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1).half().cuda(), torch.cat([ang.sin(), ang.sin()], -1).half().cuda()
    k_cache = (torch.randn(b, nkv, s, dh, generator=g) * 0.5).half().cuda()
    v_cache = torch.randn(b, nkv, s, dh, generator=g).half().cuda()
    k_cache[:, :, pos_v] = float("nan")  # stale rows at the new position must not be read
    v_cache[:, :, pos_v] = float("nan")
    k1, v1 = k_cache.clone(), v_cache.clone()
    pos = torch.tensor([pos_v], dtype=torch.long, device="cuda")
    # separate kernels
    q_out = torch.empty(b, nq, dh, dtype=torch.float16, device="cuda")
    rc.qk_rope_cache(qkv, qn, kn, cos, sin, pos, q_out, k1, v1, 1e-6, 0)
    ref_out = torch.empty(b, nq * dh, dtype=torch.float16, device="cuda")
    rc.attn_decode(q_out, k1, v1, pos, rc.attn_decode_scratch(b, nq, dh, s, "cuda"), ref_out, dh ** -0.5, 0)
    # one launch, twice on the same scratch (the arrival counters return to zero)
    scratch = rc.rope_attn_scratch(b, nq, nkv, dh, s, "cuda")
    out = torch.empty(b, nq * dh, dtype=torch.float16, device="cuda")
    for _ in range(2):
        k2, v2 = k_cache.clone(), v_cache.clone()
        out.fill_(float("nan"))
        rc.rope_attn_decode(qkv, qn, kn, cos, sin, pos, k2, v2, scratch, out, nq, dh ** -0.5, 1e-6, _lib.RDQ_GEMV_PDL)
        assert torch.equal(k2, k1) and torch.equal(v2, v1)
        _close(out, ref_out)
    mask = (torch.arange(s, device="cuda") <= pos_v)[None, None, None, :]
    ref = F.scaled_dot_product_attention(q_out[:, :, None, :].float(), k1.float(), v1.float(), attn_mask=mask, enable_gqa=True)
    _close(out, ref.reshape(b, nq * dh))
    nbytes = (b * nkv * 4 + 255) // 256 * 256
    assert int(scratch.view(torch.int32)[: nbytes // 4].abs().sum()) == 0


def test_rope_attn_decode_refuses_what_it_cannot_run():
    f16 = dict(dtype=torch.float16, device="cuda")
    pos = torch.zeros(1, dtype=torch.long, device="cuda")

    def call(nq, nkv, dh, s=64, qkv_cols=None):
        qkv = torch.zeros(1, qkv_cols or (nq + 2 * nkv) * dh, **f16)
        cos = torch.zeros(s, dh, **f16)
        kc = torch.zeros(1, nkv, s, dh, **f16)
        out = torch.zeros(1, nq * dh, **f16)
        scratch = torch.zeros(1 << 16, dtype=torch.float32, device="cuda")
        rc.rope_attn_decode(qkv, None, None, cos, cos, pos, kc, kc.clone(), scratch, out, nq, 1.0, 1e-6)

    call(4, 2, 64)  # fine
    with pytest.raises(RuntimeError, match="head_dim"):
        call(4, 2, 96)
    with pytest.raises(RuntimeError, match="query heads per KV head"):
        call(34, 2, 64)
    with pytest.raises(RuntimeError):
        call(4, 2, 64, qkv_cols=100)
