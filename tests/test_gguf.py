"""GGUF checkpoints (runtime/gguf.py): container round trip, block dequantisers, name / permutation mapping, and a
model compiled and served from a ``.gguf`` file giving the logits of its safetensors twin.
Reference: crates/plowrt/src/asset/gguf.rs."""
import glob

import numpy as np
import pytest
import torch

from plow_b200.runtime import gguf


def test_container_round_trip_and_metadata(tmp_path):
    torch.manual_seed(0)
    tensors = {"a.weight": torch.randn(6, 64), "b.weight": torch.randn(4, 32).half(), "c.weight": torch.randn(3, 32).bfloat16(),
               "scalarish": torch.arange(5, dtype=torch.float32)}
    md = {"general.architecture": "llama", "llama.block_count": 2, "some.float": 0.5, "some.flag": True, "neg": -3,
          "tokenizer.ggml.tokens": ["<s>", "</s>", "hé"], "ints": [1, 2, 3], "floats": [0.25, 0.5]}
    gguf.write_gguf(tmp_path / "t.gguf", md, tensors)
    g = gguf.GgufFile(tmp_path / "t.gguf")
    assert g.version == 3 and g.alignment == 32 and g.data_start % 32 == 0
    assert g.metadata["llama.block_count"] == 2 and g.metadata["some.flag"] is True and g.metadata["neg"] == -3
    assert g.metadata["tokenizer.ggml.tokens"] == ["<s>", "</s>", "hé"] and g.metadata["ints"] == [1, 2, 3]
    assert g.metadata["some.float"] == pytest.approx(0.5) and g.metadata["floats"] == pytest.approx([0.25, 0.5])
    for k, t in tensors.items():
        got = g.tensor(k)
        assert got.dtype == t.dtype and tuple(got.shape) == tuple(t.shape) and torch.equal(got, t)
    assert torch.equal(g.tensor("a.weight", rows=slice(2, 5)), tensors["a.weight"][2:5])
    with pytest.raises(KeyError):
        g.tensor("missing")
    (tmp_path / "bad.gguf").write_bytes(b"GGML" + b"\0" * 64)
    with pytest.raises(gguf.GgufError):
        gguf.GgufFile(tmp_path / "bad.gguf")
    blob = (tmp_path / "t.gguf").read_bytes()
    (tmp_path / "cut.gguf").write_bytes(blob[:len(blob) - 200])
    with pytest.raises(gguf.GgufError, match="past the end"):
        gguf.GgufFile(tmp_path / "cut.gguf")


def test_block_quantised_types_decode_to_their_definition(tmp_path):
    torch.manual_seed(1)
    w = torch.randn(8, 96)
    gguf.write_gguf(tmp_path / "q.gguf", {"general.architecture": "llama"}, {"q8": w, "q4": w}, types={"q8": "Q8_0", "q4": "Q4_0"})
    g = gguf.GgufFile(tmp_path / "q.gguf")
    assert g.tensors["q8"].nbytes == 8 * 96 // 32 * 34 and g.tensors["q4"].nbytes == 8 * 96 // 32 * 18
    q8, q4 = g.tensor("q8"), g.tensor("q4")
    blk = w.view(-1, 32)
    # Q8_0: scale = amax / 127 (stored as f16), value = round(x / scale) * scale
    d8 = (blk.abs().amax(1, keepdim=True) / 127).half().float()
    assert torch.allclose(q8.view(-1, 32), torch.round(blk / (blk.abs().amax(1, keepdim=True) / 127)).clamp(-127, 127) * d8, atol=1e-6)
    assert (q8 - w).abs().max() < 0.02 * w.abs().max()
    # Q4_0: 16 levels around a signed scale: coarse, but every value within one step of its source
    step = (blk.abs().amax(1, keepdim=True) / 8)
    assert ((q4.view(-1, 32) - blk).abs() <= step * 1.01 + 1e-3).all()
    # decoding a row range touches only those rows' blocks
    assert torch.equal(g.tensor("q8", rows=slice(3, 6)), q8[3:6])
    with pytest.raises(gguf.GgufError, match="multiple of the Q8_0 block"):
        gguf.write_gguf(tmp_path / "odd.gguf", {}, {"x": torch.randn(2, 40)}, types={"x": "Q8_0"})


def test_names_and_the_qk_row_permutation():
    assert gguf.hf_name("blk.7.attn_q.weight") == "model.layers.7.self_attn.q_proj.weight"
    assert gguf.hf_name("blk.0.ffn_down.weight") == "model.layers.0.mlp.down_proj.weight"
    assert gguf.hf_name("token_embd.weight") == "model.embed_tokens.weight" and gguf.hf_name("rope_freqs.weight") is None
    w = torch.arange(4 * 8 * 3, dtype=torch.float32).view(32, 3)          # 4 heads of 8 rows
    p = gguf.permute_qk(w, 4)
    assert not torch.equal(p, w) and torch.equal(gguf.unpermute_qk(p, 4), w)
    # within a head the two rotary halves are interleaved: row i of the first half lands at 2i, of the second at 2i + 1
    assert torch.equal(p[0], w[0]) and torch.equal(p[1], w[4]) and torch.equal(p[2], w[1])


def _to_gguf(ckpt_dir, cfg, path, types=None):
    """A llama.cpp-style export of a Hugging Face checkpoint: names mapped, q / k rows permuted, metadata from config."""
    from safetensors.torch import load_file
    state = {}
    for f in glob.glob(str(ckpt_dir / "*.safetensors")):
        state.update(load_file(f))
    inv_layer = {v: k for k, v in gguf._LAYER.items()}
    inv_top = {v: k for k, v in gguf._TOP.items()}
    out = {}
    for name, t in state.items():
        if name in inv_top:
            out[inv_top[name]] = t
            continue
        p = name.split(".")            # model.layers.N.<module...>.weight
        n, mod = p[2], ".".join(p[3:-1])
        if mod == "self_attn.q_proj":
            t = gguf.permute_qk(t, cfg["num_attention_heads"])
        elif mod == "self_attn.k_proj":
            t = gguf.permute_qk(t, cfg["num_key_value_heads"])
        out[f"blk.{n}.{inv_layer[mod]}.{p[-1]}"] = t
    md = {"general.architecture": "llama", "llama.block_count": cfg["num_hidden_layers"], "llama.embedding_length": cfg["hidden_size"],
          "llama.attention.head_count": cfg["num_attention_heads"], "llama.attention.head_count_kv": cfg["num_key_value_heads"],
          "llama.attention.key_length": cfg["head_dim"], "llama.feed_forward_length": cfg["intermediate_size"],
          "llama.attention.layer_norm_rms_epsilon": cfg["rms_norm_eps"], "llama.rope.freq_base": cfg["rope_theta"],
          "llama.context_length": cfg["max_position_embeddings"], "llama.vocab_size": cfg["vocab_size"],
          "tokenizer.ggml.eos_token_id": cfg["eos_token_id"], "tokenizer.ggml.bos_token_id": cfg["bos_token_id"],
          "plow.dtype": "f32", "plow.kv_dtype": "f32"}
    gguf.write_gguf(path, md, out, types=types)


def test_model_served_from_a_gguf_file_matches_its_safetensors_twin(tiny_assets, tmp_path):
    from plow_b200 import plowc
    from plow_b200.models import config
    from plow_b200.runtime.cpu_engine import CpuEngine
    from plow_b200.runtime.engine import TokenBatch
    cfg = config.tiny_dense_config()
    _to_gguf(tiny_assets / "ckpt", cfg, tmp_path / "tiny.gguf")
    spec = config.load_spec(tmp_path / "tiny.gguf")
    want = config.spec_from_config(cfg)
    assert (spec.hidden, spec.n_layers, spec.vocab, spec.tie_embeddings, spec.dtype, spec.kv_dtype) == \
        (want.hidden, want.n_layers, want.vocab, True, "f32", "f32")
    assert spec.layers[0].attn.n_kv_heads == 2 and spec.layers[0].attn.head_dim == 64 and spec.eos_token_ids == [2]
    plowc.compile_dir(tmp_path / "tiny.gguf", tmp_path / "assets", arch="cpu", n_cu=8, max_rows=256, decode_rungs=[1, 2, 4, 8], max_seqs=8)
    a = CpuEngine(tiny_assets / "assets", max_slots=2, max_ctx=256)
    b = CpuEngine(tmp_path / "assets", max_slots=2, max_ctx=256)
    rng = np.random.default_rng(0)
    p = rng.integers(0, 32000, 50).tolist()
    outs = []
    for eng in (a, b):
        eng.begin_slot(0, p)
        eng.reserve(0, 60)
        r = eng.step(TokenBatch(np.asarray(p, np.int32), np.arange(50, dtype=np.int32), np.zeros(50, np.int32), np.asarray([49], np.int32),
                                want_logits=True))
        outs.append(r.logits[0])
        eng.close()
    assert np.abs(outs[0] - outs[1]).max() < 1e-5 and int(outs[0].argmax()) == int(outs[1].argmax())
    # the same model with Q8_0 projections: close, not equal
    (tmp_path / "q8").mkdir()
    _to_gguf(tiny_assets / "ckpt", cfg, tmp_path / "q8" / "tiny-q8.gguf",
             types={f"blk.{n}.{m}.weight": "Q8_0" for n in range(4) for m in ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")})
    plowc.compile_dir(tmp_path / "q8", tmp_path / "assets_q8", arch="cpu", n_cu=8, max_rows=256, decode_rungs=[1], max_seqs=8)   # a directory holding one .gguf
    c = CpuEngine(tmp_path / "assets_q8", max_slots=2, max_ctx=256)
    c.begin_slot(0, p)
    c.reserve(0, 60)
    r = c.step(TokenBatch(np.asarray(p, np.int32), np.arange(50, dtype=np.int32), np.zeros(50, np.int32), np.asarray([49], np.int32), want_logits=True))
    c.close()
    rel = np.linalg.norm(r.logits[0] - outs[0]) / np.linalg.norm(outs[0])
    assert 0 < rel < 0.05
