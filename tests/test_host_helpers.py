"""Host-side helpers that need no GPU: the measurement decoder's per-format channel counts, its
grouped channel order, and the reader of the tiled-layout side file of a checkpoint."""
import os

import torch

from rdquant_b200.decoder import LLAMA3_70B, QWEN3_4B, DecoderConfig, MixedDecoder, _splits
from rdquant_b200.integrations import hf_export
from rdquant_b200.synthetic import fixed_splits


def test_decoder_splits_follow_the_block_benchmark():
    # the Qwen3-4B-shaped stack uses the 67 / 32 / 1 split of the block benchmark
    for n in (1024, 2560, 4096, 9728):
        assert _splits(n, QWEN3_4B) == fixed_splits(n)
    for cfg, ns in ((QWEN3_4B, (1024, 2560, 4096, 9728, 256, 48)), (LLAMA3_70B, (1024, 8192, 28672))):
        for n in ns:
            sp = _splits(n, cfg)
            assert sum(sp.values()) == n and min(sp.values()) >= 0
            unit = 128 if n >= 384 else 16
            assert all(v % unit == 0 for v in (sp["NVFP4"], sp["FP16"]))
    assert _splits(8192, LLAMA3_70B)["FP16"] == 0  # 85 / 15 NVFP4 / FP8


def test_decoder_channel_order_is_grouped_and_monotone():
    """Random assignment of channels to formats, grouped by format, original order inside a group
    (rdquant/core/allocator.py:210-224)."""
    dec = MixedDecoder.__new__(MixedDecoder)  # only the helper is exercised: no device needed
    dec.device, dec.random_perm = torch.device("cpu"), False
    gen = torch.Generator().manual_seed(3)
    sp = {"NVFP4": 640, "FP8": 256, "FP16": 128}
    perm = dec._permutation(1024, sp, gen)
    assert sorted(perm.tolist()) == list(range(1024))
    off = 0
    for fmt in ("NVFP4", "FP8", "FP16"):
        part = perm[off:off + sp[fmt]]
        assert torch.equal(part, part.sort().values)
        off += sp[fmt]
    assert not torch.equal(perm, torch.arange(1024))
    dec.random_perm = True
    shuffled = dec._permutation(1024, sp, gen)
    assert sorted(shuffled.tolist()) == list(range(1024))
    assert not torch.equal(shuffled[:640], shuffled[:640].sort().values)


def test_decoder_config_shapes():
    assert QWEN3_4B.layers == 36 and QWEN3_4B.hidden == 2560 and QWEN3_4B.q_heads * QWEN3_4B.head_dim == 4096
    assert LLAMA3_70B.layers == 80 and LLAMA3_70B.q_heads // LLAMA3_70B.kv_heads == 8
    assert isinstance(DecoderConfig(), DecoderConfig)


def test_tiled_layout_file_reader(tmp_path):
    from safetensors.torch import save_file

    assert hf_export.read_tiled_layout(str(tmp_path)) == {}  # no file
    blob = {"model.layers.0.mlp.down_proj.weight_tiled": torch.arange(64, dtype=torch.uint8)}
    save_file(blob, os.path.join(tmp_path, hf_export.TILED_FILE), metadata={"layout": hf_export.TILED_LAYOUT})
    got = hf_export.read_tiled_layout(str(tmp_path))
    assert list(got) == list(blob) and torch.equal(got[list(blob)[0]], blob[list(blob)[0]])
    save_file(blob, os.path.join(tmp_path, hf_export.TILED_FILE), metadata={"layout": "another version"})
    assert hf_export.read_tiled_layout(str(tmp_path)) == {}
    save_file(blob, os.path.join(tmp_path, hf_export.TILED_FILE))  # no metadata at all
    assert hf_export.read_tiled_layout(str(tmp_path)) == {}
