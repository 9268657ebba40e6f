"""The measurement decoder (rdquant_b200.decoder) on a tiny configuration: a CUDA-graph replay of
the decode step produces the same tokens as the eager step, prefill through the GEMM path and
decode through the GEMV path agree on the next token, and the linears inside it match dense
linears holding the dequantised weights."""
import pytest
import torch

from rdquant_b200.decoder import DecoderConfig, MixedDecoder

pytestmark = pytest.mark.gpu

TINY = DecoderConfig(layers=2, hidden=256, ffn=512, q_heads=4, kv_heads=2, head_dim=64, vocab=1024, name="tiny")


def _generate(model, ids, steps, graph):
    model.reset(ids.shape[0])
    out = [model.prefill(ids)]
    if graph:
        model.capture_decode()
    for _ in range(steps):
        model.decode_step()
        out.append(model.ids.clone())
    return torch.stack(out, dim=1)


def test_graph_replay_matches_eager_decode():
    model = MixedDecoder(TINY, "cuda", max_seq=64, batch=2, seed=3)
    ids = torch.randint(0, TINY.vocab, (2, 20), generator=torch.Generator().manual_seed(1)).cuda()
    eager = _generate(model, ids, 6, graph=False)
    graphed = _generate(model, ids, 6, graph=True)
    assert torch.equal(eager, graphed)
    assert int(model.pos) == 26


def test_fused_glue_step_matches_framework_step():
    """The decode step over the glue kernels gives the logits of the step over PyTorch operators."""
    model = MixedDecoder(TINY, "cuda", max_seq=64, batch=3, seed=5)
    ids = torch.randint(0, TINY.vocab, (3, 17), generator=torch.Generator().manual_seed(3)).cuda()
    model.prefill(ids)
    caches = [(b["k"].clone(), b["v"].clone()) for b in model.blocks]
    with torch.no_grad():
        ref = model._forward(model.ids[:, None], 1, model.pos).float()
        for b, (k, v) in zip(model.blocks, caches):
            b["k"].copy_(k)
            b["v"].copy_(v)
        got = model._forward_fused().float()
    err = (got - ref).abs().max() / ref.abs().max()
    assert float(err) < 1e-2, float(err)
    for b in model.blocks:  # both paths wrote the same cache rows
        assert float((b["k"][:, :, 17].float() - b["k"][:, :, 17].float()).abs().max()) == 0.0


def test_prefill_and_decode_paths_agree():
    """Feeding the prompt token by token through the decode path (GEMV, M = 1) ends in the same
    logits as one prefill pass (GEMM, M = 20)."""
    model = MixedDecoder(TINY, "cuda", max_seq=64, batch=1, seed=4)
    ids = torch.randint(0, TINY.vocab, (1, 20), generator=torch.Generator().manual_seed(2)).cuda()
    with torch.no_grad():
        full = model._forward(ids, 20, 0).float()
        model.reset(1)
        for t in range(20):
            step = model._forward(ids[:, t:t + 1], 1, t).float()
    err = (full - step).abs().max() / full.abs().max()
    assert float(err) < 2e-2, float(err)


@pytest.mark.parametrize("batch", [1, 4])
def test_prologue_fusion_matches_separate_glue_kernels(batch):
    """Norms and SiLU x mul folded into the consuming GEMV give the logits of the step that runs
    them as separate kernels (the mean square is summed in another order: last-bit differences)."""
    ids = torch.randint(0, TINY.vocab, (batch, 11), generator=torch.Generator().manual_seed(7)).cuda()
    logits = []
    for fuse in (True, False):
        model = MixedDecoder(TINY, "cuda", max_seq=64, batch=batch, seed=9, fuse_prologue=fuse)
        model.prefill(ids)
        with torch.no_grad():
            logits.append(model._forward_fused().float())
    err = (logits[0] - logits[1]).abs().max() / logits[1].abs().max()
    assert float(err) < 5e-3, float(err)
