"""The GGUF reader and the dense-decoder model view, on the host (no GPU): files written here,
read back through libapk_b200.so.  Mirrors the reference's own header tests
(crates/allpaka-gguf/src/metadata.rs:595-745) and loader checks (crates/allpaka-model/src/model/
loader.rs:366-426, 558-580; config.rs:184-310)."""
import ctypes as C
import struct

import numpy as np
import pytest

from allpaka_b200 import gguf, synth
from tests.util import Q4_K, Q6_K, Q8_0


@pytest.fixture(scope="module", autouse=True)
def _library():
    from allpaka_b200 import build

    build.build()  # (no-op when the library is up to date)


def tiny_model(arch="qwen3", ty=Q8_0, hidden=256, n_heads=2, n_kv=1, head_dim=128, ffn=512, vocab=300, n_layers=2,
               qk_norm=True, tied=False, extra_meta=None, drop=(), override=None, ty_of=None):
    """ty_of: tensor-name suffix -> ggml type, for files that mix types (the rest take ``ty``)."""
    rng = np.random.default_rng(3)
    meta = {"general.architecture": arch, f"{arch}.block_count": n_layers, f"{arch}.embedding_length": hidden,
            f"{arch}.attention.head_count": n_heads, f"{arch}.attention.head_count_kv": n_kv,
            f"{arch}.attention.key_length": head_dim, f"{arch}.feed_forward_length": ffn,
            f"{arch}.attention.layer_norm_rms_epsilon": 1e-6, f"{arch}.rope.freq_base": 1e6,
            "tokenizer.ggml.tokens": [f"t{i}" for i in range(vocab)], "tokenizer.ggml.scores": [1, 2, 3]}
    meta.update(extra_meta or {})
    q_dim, kv_dim = n_heads * head_dim, n_kv * head_dim

    def mat(name, n_out, n_in, seed):
        t_ = next((v for k, v in (ty_of or {}).items() if name.endswith(k)), ty)
        return (name, t_, [n_in, n_out], synth.matrix(t_, n_out, n_in, seed))

    t = [mat("token_embd.weight", vocab, hidden, 1)]
    for l in range(n_layers):
        def vec(n, s):
            return (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        t += [(f"blk.{l}.attn_norm.weight", 0, [hidden], vec(hidden, 0)),
              mat(f"blk.{l}.attn_q.weight", q_dim, hidden, 10 * l + 2),
              mat(f"blk.{l}.attn_k.weight", kv_dim, hidden, 10 * l + 3),
              mat(f"blk.{l}.attn_v.weight", kv_dim, hidden, 10 * l + 4),
              mat(f"blk.{l}.attn_output.weight", hidden, q_dim, 10 * l + 5),
              (f"blk.{l}.ffn_norm.weight", 0, [hidden], vec(hidden, 1)),
              mat(f"blk.{l}.ffn_gate.weight", ffn, hidden, 10 * l + 6),
              mat(f"blk.{l}.ffn_up.weight", ffn, hidden, 10 * l + 7),
              mat(f"blk.{l}.ffn_down.weight", hidden, ffn, 10 * l + 8)]
        if qk_norm:
            t += [(f"blk.{l}.attn_q_norm.weight", 0, [head_dim], vec(head_dim, 2)),
                  (f"blk.{l}.attn_k_norm.weight", 0, [head_dim], vec(head_dim, 3))]
    t.append(("output_norm.weight", 0, [hidden], (1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)))
    if not tied:
        t.append(mat("output.weight", vocab, hidden, 99))
    t = [e for e in t if e[0] not in drop]
    if override:
        t = [override.get(e[0], e) for e in t]
    return meta, t


def test_round_trip_of_metadata_and_tensor_bytes(tmp_path):
    meta, tensors = tiny_model()
    for alignment, version in ((32, 3), (64, 2)):
        p = tmp_path / f"m{alignment}.gguf"
        gguf.write_file(str(p), meta, tensors, alignment=alignment, version=version)
        f = gguf.GgufFile(str(p))
        assert f.architecture == "qwen3"
        assert f.meta_u32("qwen3.block_count") == 2 and f.meta_u32("qwen3.missing") is None
        assert abs(f.meta_f32("qwen3.rope.freq_base") - 1e6) < 1 and f.meta_f32("qwen3.block_count") is None
        assert f.meta_str("general.architecture") == "qwen3"
        got = {t["name"]: t for t in f.tensors()}
        assert list(got) == [t[0] for t in tensors]  # file order
        base = f.mapping().ctypes.data
        for name, ty, dims, data in tensors:
            g = got[name]
            assert g["ty"] == ty and g["dims"] == list(dims)
            assert np.array_equal(g["data"], np.asarray(data).reshape(-1).view(np.uint8))
            assert (g["data"].ctypes.data - base) % alignment == 0
        assert f.tensor("blk.1.ffn_up.weight")["dims"] == [256, 512] and f.tensor("nope") is None
        f.close()


def test_malformed_files_are_rejected(tmp_path):
    meta, tensors = tiny_model(n_layers=1)
    good = tmp_path / "good.gguf"
    gguf.write_file(str(good), meta, tensors)
    raw = good.read_bytes()

    def expect(name, data, what):
        p = tmp_path / name
        p.write_bytes(data)
        with pytest.raises(gguf.GgufError) as e:
            gguf.GgufFile(str(p))
        assert what in str(e.value), str(e.value)

    expect("magic.gguf", b"GGML" + raw[4:], "magic")                       # a_non_gguf_file_is_rejected
    expect("v1.gguf", raw[:4] + struct.pack("<I", 1) + raw[8:], "version 1")
    expect("short.gguf", raw[:200], "truncated")
    expect("cut.gguf", raw[:len(raw) - 4096], "but the file has only")       # tensor bytes past the end
    five = bytearray(raw)
    at = raw.index(b"token_embd.weight") + len(b"token_embd.weight")
    five[at:at + 4] = struct.pack("<I", 5)
    expect("five.gguf", bytes(five), "at most 4")
    with pytest.raises(gguf.GgufError):
        gguf.GgufFile(str(tmp_path / "absent.gguf"))


def test_model_view_binds_checked_tensors(tmp_path):
    meta, tensors = tiny_model(ty=Q4_K, tied=True)
    p = tmp_path / "m.gguf"
    gguf.write_file(str(p), meta, tensors)
    f = gguf.GgufFile(str(p))
    m = gguf.Model(f)
    assert m.info == {"n_layers": 2, "hidden": 256, "n_heads": 2, "n_kv_heads": 1, "head_dim": 128, "ffn": 512, "vocab": 300,
                      "rot_dim": 128, "eps": pytest.approx(1e-6), "rope_base": pytest.approx(1e6), "has_qk_norm": 1,
                      "neox_reordered": 0, "tied": 1}
    r = m.request()
    assert (r.n_layers, r.hidden, r.head_dim, r.n_heads, r.n_kv_heads, r.rot_dim, r.m) == (2, 256, 128, 2, 1, 128, 1)
    assert r.attn_core == 2 and r.scale == pytest.approx(128 ** -0.5)
    # the request points straight into the mapping
    assert r.output.w == f.tensor("token_embd.weight")["data"].ctypes.data and r.embd.w == r.output.w and r.output.n_out == 300
    L1 = m.layer(1)
    assert L1.wq.w == f.tensor("blk.1.attn_q.weight")["data"].ctypes.data and L1.wq.ty == Q4_K and L1.wq.n_out == 256
    assert L1.down.w == f.tensor("blk.1.ffn_down.weight")["data"].ctypes.data and L1.down.n_out == 256
    assert L1.q_norm == f.tensor("blk.1.attn_q_norm.weight")["data"].ctypes.data
    assert L1.ffn_norm == f.tensor("blk.1.ffn_norm.weight")["data"].ctypes.data
    m.close()
    f.close()


def test_head_dim_is_implied_and_block_count_is_trimmed(tmp_path):
    """config.rs:224-228 (key_length absent -> hidden / heads), 258-264 (blocks without tensors are trimmed)."""
    meta, tensors = tiny_model(hidden=256, n_heads=2, head_dim=128, qk_norm=False)
    del meta["qwen3.attention.key_length"]
    meta["qwen3.block_count"] = 3  # one more than the file carries
    p = tmp_path / "m.gguf"
    gguf.write_file(str(p), meta, tensors)
    f = gguf.GgufFile(str(p))
    m = gguf.Model(f)
    assert m.info["head_dim"] == 128 and m.info["n_layers"] == 2 and m.info["has_qk_norm"] == 0 and m.info["tied"] == 0
    m.close()
    f.close()


def test_pairwise_rope_files_get_their_q_and_k_rows_reordered(tmp_path):
    """neox_order + reorder_head_rows (loader.rs:366-426): new row i of a head is old row 2i (first half)
    or 2(i - half) + 1 (second half); whole quantised rows move, V and the other matrices stay."""
    for ty in (Q8_0, Q6_K):
        meta, tensors = tiny_model(arch="llama", ty=ty, qk_norm=False)
        p = tmp_path / f"l{ty}.gguf"
        gguf.write_file(str(p), meta, tensors)
        f = gguf.GgufFile(str(p))
        m = gguf.Model(f)
        assert m.info["neox_reordered"] == 1
        order = [2 * i for i in range(64)] + [2 * i + 1 for i in range(64)]
        row = synth.expected_bytes(ty, 256)
        for part, field, n_heads in (("attn_q", "wq", 2), ("attn_k", "wk", 1)):
            src = f.tensor(f"blk.1.{part}.weight")["data"].reshape(n_heads, 128, row)
            want = src[:, order, :].reshape(-1)
            mat = getattr(m.layer(1), field)
            got = np.ctypeslib.as_array(C.cast(mat.w, C.POINTER(C.c_uint8)), shape=(want.size,))
            assert np.array_equal(got, want)
        assert m.layer(1).wv.w == f.tensor("blk.1.attn_v.weight")["data"].ctypes.data
        m.close()
        f.close()


def test_pairwise_rope_kept_in_file_order_is_declined(tmp_path, monkeypatch):
    """neox_order returns None for per-head norms or ALLPAKA_ROPE_NORM=1 (loader.rs:366-375): the reference then
    rotates adjacent pairs at run time, which the kernels here do not."""
    meta, tensors = tiny_model(arch="llama", qk_norm=False)
    p = tmp_path / "l.gguf"
    gguf.write_file(str(p), meta, tensors)
    f = gguf.GgufFile(str(p))
    monkeypatch.setenv("ALLPAKA_ROPE_NORM", "1")
    with pytest.raises(gguf.GgufError) as e:
        gguf.Model(f)
    assert "pairwise rotary" in str(e.value) and e.value.rc == 5
    monkeypatch.delenv("ALLPAKA_ROPE_NORM")
    gguf.Model(f).close()
    f.close()
    meta, tensors = tiny_model(arch="mistral", qk_norm=True)
    gguf.write_file(str(p), meta, tensors)
    f = gguf.GgufFile(str(p))
    with pytest.raises(gguf.GgufError):
        gguf.Model(f)
    f.close()


def test_what_the_decode_path_cannot_serve_is_declined_by_name(tmp_path):
    def fails(what, **kw):
        meta, tensors = tiny_model(**kw)
        p = tmp_path / "bad.gguf"
        gguf.write_file(str(p), meta, tensors)
        f = gguf.GgufFile(str(p))
        with pytest.raises(gguf.GgufError) as e:
            gguf.Model(f)
        assert what in str(e.value), str(e.value)
        f.close()

    w = synth.matrix(Q8_0, 256, 256, 5)
    fails('"blk.0.attn_q.weight" has shape [128, 512], expected [256, 256]',   # a transposed / misshapen tensor is named
          override={"blk.0.attn_q.weight": ("blk.0.attn_q.weight", Q8_0, [128, 512], w)})
    fails('no tensor "blk.1.ffn_down.weight"', drop=("blk.1.ffn_down.weight",))
    fails("is not F32", override={"blk.0.attn_norm.weight": ("blk.0.attn_norm.weight", 1, [256], np.zeros(256, np.float16))})
    fails("mixture-of-experts", extra_meta={"qwen3.expert_count": 8})
    fails("has no kernel", override={"blk.0.ffn_up.weight": ("blk.0.ffn_up.weight", 2, [256, 512], np.zeros(512 * 256 // 32 * 18, np.uint8))})
    meta, tensors = tiny_model()
    del meta["qwen3.block_count"]                                            # a_model_without_block_count_is_rejected
    p = tmp_path / "nb.gguf"
    gguf.write_file(str(p), meta, tensors)
    f = gguf.GgufFile(str(p))
    with pytest.raises(gguf.GgufError) as e:
        gguf.Model(f)
    assert "qwen3.block_count" in str(e.value)
    f.close()
