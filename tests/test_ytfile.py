"""`.yt` container: files written by the reference's yt::io::YTensorIO are read back exactly, files written here
keep their contents, malformed files are refused, and a converted-checkpoint file loads into the decoder layout."""
import struct
from pathlib import Path

import numpy as np
import pytest

from ytensor_b200 import ytfile
from ytensor_b200.qwen3 import Qwen3Config, random_weights

GOLDEN = Path(__file__).resolve().parent / "golden"
SMALL = dict(hidden_size=64, num_hidden_layers=2, vocab_size=512, intermediate_size=96, num_attention_heads=4,
             num_key_value_heads=2, head_dim=128, max_position_embeddings=64)


@pytest.mark.parametrize("fname,method", [("ref_sample.yt", ""), ("ref_sample_zlib.yt", "zlib")])
def test_reads_files_written_by_the_reference(fname, method):
    want = np.load(GOLDEN / "golden_yt.npz")
    with ytfile.YtFile(GOLDEN / fname) as f:
        assert f.names() == ["weights.f32", "weights.bf16", "ids", "tiled.f32"]
        for name in f.names():
            r = f.record(name)
            assert r.compress == method and r.tensor_type == "dense"
            assert np.array_equal(f.load(name), want[name])
        assert f.record("weights.bf16").type_name == "bfloat16" and f.record("weights.bf16").type_size == 2
        assert f.record("ids").type_name == "int32" and f.record("ids").shape == (2, 3)
        with pytest.raises(KeyError):
            f.load("missing")


@pytest.mark.parametrize("method", ["", "zlib"])
def test_write_then_read(tmp_path, method):
    rng = np.random.default_rng(1)
    t = {"a": rng.standard_normal((3, 4, 5)).astype(np.float32), "b": rng.integers(0, 65535, (7, 2)).astype(np.uint16),
         "scalar_like": np.arange(6, dtype=np.int64), "empty": np.zeros((0, 4), np.float32)}
    p = tmp_path / "t.yt"
    ytfile.write_yt(p, t, compress=method, bfloat16=("b",), metadata="note")
    with ytfile.YtFile(p) as f:
        assert f.metadata == "note" and f.names() == list(t)
        for k, v in t.items():
            assert np.array_equal(f.load(k), v) and f.load(k).shape == v.shape
        assert f.record("b").type_name == "bfloat16"


def test_malformed_files_are_refused(tmp_path):
    good = (GOLDEN / "ref_sample.yt").read_bytes()
    bad_magic = tmp_path / "m.yt"
    bad_magic.write_bytes(b"NOTATENS" + good[8:])
    with pytest.raises(ytfile.YtFormatError):
        ytfile.YtFile(bad_magic)
    count_too_big = tmp_path / "c.yt"
    count_too_big.write_bytes(good[:-4] + struct.pack("<I", 1 << 20))
    with pytest.raises(ytfile.YtFormatError):
        ytfile.YtFile(count_too_big)
    cut = tmp_path / "cut.yt"   # the first tensor's data runs into the index
    cut.write_bytes(good[:60] + good[-(4 + 8 * 4):])
    with pytest.raises(ytfile.YtFormatError):
        ytfile.YtFile(cut)
    with pytest.raises(ValueError):
        ytfile.write_yt(tmp_path / "x.yt", {"a": np.zeros(3, np.complex64)})


def _checkpoint_tensors(cfg, w):
    """The tensors a converted checkpoint holds (names of qwen3.cpp:304-364), from the fused layout."""
    D, H, KV, I = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size
    t, bf = {"model.embed_tokens.weight": w["embed"], "model.norm.weight": w["norm"]}, ["model.embed_tokens.weight"]
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        qkv, gu = w[("qkv", l)], w[("gate_up", l)]
        mats = {"self_attn.q_proj.weight": qkv[:H * D], "self_attn.k_proj.weight": qkv[H * D:(H + KV) * D],
                "self_attn.v_proj.weight": qkv[(H + KV) * D:], "self_attn.o_proj.weight": w[("o", l)],
                "mlp.gate_proj.weight": gu[:I], "mlp.up_proj.weight": gu[I:], "mlp.down_proj.weight": w[("down", l)]}
        for k, v in mats.items():
            t[p + k] = v
            bf.append(p + k)
        t[p + "self_attn.q_norm.weight"], t[p + "self_attn.k_norm.weight"] = w[("q_norm", l)], w[("k_norm", l)]
        t[p + "input_layernorm.weight"], t[p + "post_attention_layernorm.weight"] = w[("norm1", l)], w[("norm2", l)]
    return t, tuple(bf)


def test_checkpoint_loader_rebuilds_the_fused_layout(tmp_path):
    cfg = Qwen3Config(**SMALL)
    w = random_weights(cfg, seed=9, std=0.05)
    w[("norm1", 1)] = np.linspace(0.5, 1.5, cfg.hidden_size).astype(np.float32)
    t, bf = _checkpoint_tensors(cfg, w)
    p = tmp_path / "ckpt.yt"
    ytfile.write_yt(p, t, compress="zlib", bfloat16=bf)
    got = ytfile.load_qwen3_checkpoint(p, cfg)
    assert set(got) == set(w)
    for k in w:
        assert np.array_equal(got[k], w[k]), k
    # a matrix stored as float32 is refused: the device kernels stream bfloat16 weights
    t2 = dict(t)
    t2["model.layers.0.mlp.down_proj.weight"] = np.zeros((cfg.hidden_size, cfg.intermediate_size), np.float32)
    ytfile.write_yt(p, t2, bfloat16=tuple(b for b in bf if b != "model.layers.0.mlp.down_proj.weight"))
    with pytest.raises(ytfile.YtFormatError):
        ytfile.load_qwen3_checkpoint(p, cfg)


@pytest.mark.gpu
def test_decoder_loaded_from_yt_matches_decoder_loaded_from_arrays(tmp_path):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from ytensor_b200 import qwen3 as Q
    cfg = Qwen3Config(**SMALL)
    w = random_weights(cfg, seed=9, std=0.05)
    t, bf = _checkpoint_tensors(cfg, w)
    p = tmp_path / "ckpt.yt"
    ytfile.write_yt(p, t, bfloat16=bf)
    ids = torch.from_numpy(np.random.default_rng(2).integers(0, cfg.vocab_size, (2, 11)).astype(np.int32)).cuda()
    outs = []
    for weights in (w, ytfile.load_qwen3_checkpoint(p, cfg)):
        m = Q.Qwen3ForCausalLM(cfg, batch=2)
        m.load_weights(weights)
        logits = m.forward(ids)
        tok, _ = m.argmax(logits)
        outs.append((logits.cpu().numpy(), m.forward(tok.reshape(2, 1).contiguous()).cpu().numpy()))
        m.close()
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    with ytfile.YtFile(p) as f:
        e = f.to_device("model.embed_tokens.weight")
        assert e.dtype == torch.bfloat16 and tuple(e.shape) == (cfg.vocab_size, cfg.hidden_size)
        assert np.array_equal(e.view(torch.int16).cpu().numpy().view(np.uint16), w["embed"])


def test_unknown_compression_name_falls_back_to_none(tmp_path):
    """The reference names "zlibfloat" in a comment but implements only "" and "zlib": checkCompressMethod turns any
    other name into "no compression" (src/ytensor_io.inl:11-22). Writer and reader here do the same."""
    from ytensor_b200 import ytfile
    a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    p = tmp_path / "zf.yt"
    ytfile.write_yt(p, {"a": a}, compress="zlibfloat")
    with ytfile.YtFile(p) as f:
        assert f.record("a").compress == ""
        assert np.array_equal(f.load("a"), a)
