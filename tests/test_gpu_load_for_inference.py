"""load_for_inference on a packed checkpoint of a small random-init Qwen3 model (the reference's
counterpart: tests/test_fused_inference.py:62-89, :309-324, there with a one-layer dummy model).
The checkpoint is written by save_packed; the loaded model's logits are compared with the same
architecture carrying the dequantised weights as dense linears, for a decode-sized input (GEMV
path) and a prefill-sized one (tcgen05 GEMM path)."""
import json
import os

import pytest
import torch
import torch.nn as nn

from rdquant_b200.integrations import hf_export
from rdquant_b200.quantize import QuantizedLayer, QuantizedModel, quantize_weight

SPLITS = {128: (64, 48, 16), 256: (128, 96, 32), 512: (256, 192, 64)}
ORDER = ("NVFP4", "FP8", "FP16")


def _tiny_config():
    from transformers import Qwen3Config

    return Qwen3Config(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, head_dim=64, vocab_size=512, max_position_embeddings=128,
                       tie_word_embeddings=True, attention_bias=True)


def write_checkpoint(path: str, seed: int = 0):
    """Random-init tiny Qwen3, every decoder linear quantised (fixed splits, random permutation),
    written with save_packed + config.json.  Returns the names of the quantised layers."""
    from transformers import AutoModelForCausalLM

    torch.manual_seed(seed)
    cfg = _tiny_config()
    model = AutoModelForCausalLM.from_config(cfg)
    gen = torch.Generator().manual_seed(seed)
    names = [n for n, m in model.named_modules() if isinstance(m, nn.Linear) and ".layers." in n]
    for name in names:
        lin = model.get_submodule(name)
        n_out, n_in = lin.weight.shape
        w = lin.weight.data.half()
        perm = torch.randperm(n_out, generator=gen)
        qw = quantize_weight(w.float(), perm, dict(zip(ORDER, SPLITS[n_out])))
        bias = lin.bias.data.half() if lin.bias is not None else None
        parent = model.get_submodule(name.rsplit(".", 1)[0])
        setattr(parent, name.rsplit(".", 1)[1], QuantizedLayer(qw, bias, n_in, n_out))
    hf_export.save_packed(QuantizedModel(model, formats=list(ORDER), budget_avg_bits=5.3), path)
    cfg.save_pretrained(path)
    return names


def test_checkpoint_layout(tmp_path):
    names = write_checkpoint(str(tmp_path))
    assert len(names) == 14
    qcfg = json.load(open(os.path.join(tmp_path, "quantization_config.json")))
    assert set(qcfg["layers"]) == set(names)
    _, tensors = hf_export.read_layers(str(tmp_path))
    assert "model.embed_tokens.weight" in tensors and "model.layers.0.self_attn.q_proj.bias" in tensors
    assert tensors["model.layers.1.mlp.down_proj.weight_nvfp4"].shape == (128, 256)


@pytest.mark.gpu
def test_loaded_model_matches_dense_dequantised_model(tmp_path):
    from transformers import AutoModelForCausalLM

    from rdquant_b200 import rdquant_cuda
    from rdquant_b200.inference import FusedMixedLinear, load_for_inference

    names = write_checkpoint(str(tmp_path))
    model = load_for_inference(str(tmp_path), device="cuda")
    for name in names:
        assert isinstance(model.get_submodule(name), FusedMixedLinear), name
    assert model.lm_head.weight is model.model.embed_tokens.weight  # tie restored

    # the same architecture with dense linears holding the bit-exact dequantised weights
    qcfg, tensors = hf_export.read_layers(str(tmp_path))
    dense = AutoModelForCausalLM.from_config(_tiny_config())
    state = {k: v for k, v in tensors.items() if k in dense.state_dict()}  # (rotary tables are rebuilt from the config)
    for name in names:
        lconf = qcfg["layers"][name]
        data = {k[len(name) + 1:]: v.cuda() for k, v in tensors.items() if k.startswith(name + ".")}
        w = rdquant_cuda.dequantize_packed(data, lconf["splits"], lconf["in_features"], inv_perm=data["inv_permutation"])
        state[name + ".weight"] = w.cpu()
        if "bias" in data:
            state[name + ".bias"] = data["bias"].cpu()
    missing, unexpected = dense.load_state_dict({k: v.float() for k, v in state.items()}, strict=False)
    assert not unexpected and all("lm_head" in m for m in missing), (missing, unexpected)
    dense.lm_head.weight = dense.model.embed_tokens.weight
    dense = dense.cuda().eval()

    gen = torch.Generator().manual_seed(1)
    for tokens in (6, 40):  # M <= 16: decode GEMV; M > 16: prefill GEMM
        ids = torch.randint(0, 512, (1, tokens), generator=gen).cuda()
        with torch.no_grad():
            got = model(input_ids=ids).logits.float()
            ref = dense(input_ids=ids).logits.float()
        err = (got - ref).abs().max() / ref.abs().max()
        assert float(err) < 1e-2, (tokens, float(err))


@pytest.mark.gpu
def test_tiled_layout_in_checkpoint_is_used_as_is(tmp_path):
    """save_tiled_layout writes the decode kernel's tiling beside the checkpoint (which keeps its
    bytes); a load then uploads it instead of re-tiling, and the model computes the same logits
    bit for bit.  A file of another layout version, or a tensor of the wrong size, is ignored."""
    import hashlib

    from safetensors.torch import save_file

    from rdquant_b200.inference import load_for_inference

    names = write_checkpoint(str(tmp_path))
    main = os.path.join(tmp_path, "model.safetensors")
    sha = hashlib.sha256(open(main, "rb").read()).hexdigest()
    plain = load_for_inference(str(tmp_path), device="cuda")
    assert not any(plain.get_submodule(n)._fd().get("tiled_from_checkpoint") for n in names)

    info = hf_export.save_tiled_layout(str(tmp_path), device="cuda")
    assert info["layers"] == len(names) and info["bytes"] > 0
    assert hashlib.sha256(open(main, "rb").read()).hexdigest() == sha
    fast = load_for_inference(str(tmp_path), device="cuda")
    for n in names:
        a, b = plain.get_submodule(n)._fd(), fast.get_submodule(n)._fd()
        assert b.get("tiled_from_checkpoint") and torch.equal(a["w_tiled"], b["w_tiled"]), n
    ids = torch.randint(0, 512, (1, 5), generator=torch.Generator().manual_seed(2)).cuda()
    with torch.no_grad():
        assert torch.equal(plain(input_ids=ids).logits, fast(input_ids=ids).logits)

    # wrong size -> re-tiled at load; other layout version -> file ignored
    tiled = hf_export.read_tiled_layout(str(tmp_path))
    key = names[0] + ".weight_tiled"
    tiled[key] = tiled[key][:-16].contiguous()
    save_file(tiled, os.path.join(tmp_path, hf_export.TILED_FILE), metadata={"layout": hf_export.TILED_LAYOUT})
    again = load_for_inference(str(tmp_path), device="cuda")
    assert not again.get_submodule(names[0])._fd().get("tiled_from_checkpoint")
    assert again.get_submodule(names[1])._fd().get("tiled_from_checkpoint")
    assert torch.equal(again.get_submodule(names[0])._fd()["w_tiled"], plain.get_submodule(names[0])._fd()["w_tiled"])
    save_file(tiled, os.path.join(tmp_path, hf_export.TILED_FILE), metadata={"layout": "something else"})
    assert hf_export.read_tiled_layout(str(tmp_path)) == {}


@pytest.mark.gpu
def test_decode_only_load_keeps_one_copy_of_the_weights(tmp_path):
    """decode_only=True drops the row-major tensors (the tiled copy alone stays on the device):
    decode-sized inputs give the same bits as the full load, longer inputs run as 16-row panels
    of the decode kernel and agree with the tensor-core GEMM within the FP32-sum tolerance."""
    from rdquant_b200 import rdquant_cuda
    from rdquant_b200.inference import load_for_inference

    names = write_checkpoint(str(tmp_path))
    full = load_for_inference(str(tmp_path), device="cuda")
    lean = load_for_inference(str(tmp_path), device="cuda", decode_only=True)

    def weight_bytes(model):
        total = 0
        for n in names:
            fd = model.get_submodule(n)._fd()
            total += sum(fd[k].numel() * fd[k].element_size() for k in ("w_fp4_q", "w_fp4_scales", "w_fp8_q", "w_fp16", "w_tiled")
                         if fd.get(k) is not None)
        return total

    for n in names:
        fd = lean.get_submodule(n)._fd()
        assert fd["row_major"] is False and fd["w_tiled"] is not None
        assert all(fd.get(k) is None for k in ("w_fp4_q", "w_fp4_scales", "w_fp8_q", "w_fp16"))
    assert weight_bytes(lean) < 0.55 * weight_bytes(full)

    gen = torch.Generator().manual_seed(4)
    ids = torch.randint(0, 512, (1, 7), generator=gen).cuda()
    with torch.no_grad():
        assert torch.equal(full(input_ids=ids).logits, lean(input_ids=ids).logits)
        ids = torch.randint(0, 512, (1, 45), generator=gen).cuda()
        a, b = full(input_ids=ids).logits.float(), lean(input_ids=ids).logits.float()
    assert float((a - b).abs().max() / a.abs().max()) < 5e-3
    fd = lean.get_submodule(names[0])._fd()
    x = torch.zeros(32, fd["k"], dtype=torch.float16, device="cuda")
    with pytest.raises(RuntimeError, match="row-major"):
        rdquant_cuda.mixed_gemm(x, fd)
    with pytest.raises(RuntimeError, match="row-major"):
        rdquant_cuda.mixed_gemv(x[:1], fd, None, 1)  # forced any-shape kernel
