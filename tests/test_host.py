"""Host-side logic that needs no GPU: the synthetic generator, GGUF round trip, byte accounting."""
import os

import numpy as np

from nfai_b200 import gguf_io, synth


def test_tensor_streams_are_independent_and_seeded():
    cfg = synth.get_config("c0")
    a = synth.gen_tensor(cfg, "blk.1.attn_q.weight", (cfg.H, cfg.qDim), "f32", 0)
    b = synth.gen_tensor(cfg, "blk.1.attn_q.weight", (cfg.H, cfg.qDim), "f32", 0)
    c = synth.gen_tensor(cfg, "blk.0.attn_q.weight", (cfg.H, cfg.qDim), "f32", 0)
    d = synth.gen_tensor(cfg, "blk.1.attn_q.weight", (cfg.H, cfg.qDim), "f32", 1)
    assert np.array_equal(a, b) and not np.array_equal(a, c) and not np.array_equal(a, d)
    assert a.shape == (cfg.qDim, cfg.H)
    assert abs(float(a.std()) - 0.02) < 1e-3
    g = synth.gen_tensor(cfg, "blk.0.attn_norm.weight", (cfg.H,), "f32", 0)
    assert np.all(g == 1.0)


def test_prompt_ids_are_in_range():
    cfg = synth.get_config("c0")
    p = synth.prompt_ids(cfg, 64, 0)
    assert p.dtype == np.uint32 and p.shape == (64,) and p.max() < cfg.V
    assert np.array_equal(p, synth.prompt_ids(cfg, 64, 0))


def test_parameter_counts_match_the_architectures():
    assert synth.get_config("c0").streamed_matrix_params() == 2_555_904
    assert synth.get_config("c1").streamed_matrix_params() == 1_235_746_816
    assert synth.get_config("c2").streamed_matrix_params() == 3_212_574_720
    assert synth.get_config("c3").streamed_matrix_params() == 7_504_658_432


def test_decode_bytes_formula():
    cfg = synth.get_config("c1")
    b0 = synth.decode_bytes(cfg, 0, 2)
    b1 = synth.decode_bytes(cfg, 1, 2)
    assert b1 - b0 == 2 * cfg.L * cfg.kvDim * 2  # one more position of K and V to read: 32 768 B
    assert b1 - b0 == 32768
    assert abs(synth.decode_bytes(cfg, 255, 2) - 2.480e9) < 0.01e9


def test_gguf_round_trip(tmp_path):
    cfg = synth.get_config("s3")
    path = os.path.join(tmp_path, "s3.gguf")
    gguf_io.write_synthetic_gguf(cfg, path, seed=3)
    meta, tensors = gguf_io.read_gguf(path)
    assert meta["general.architecture"] == "llama"
    assert meta["llama.block_count"] == cfg.L
    assert meta["llama.attention.head_count_kv"] == cfg.kvH
    assert abs(meta["llama.rope.freq_base"] - 500000.0) < 1e-3
    want = {n: (ne, dt, a) for n, ne, dt, a in synth.iter_tensors(cfg, 3)}
    assert sorted(t.Name for t in tensors) == sorted(want)
    for t in tensors:
        ne, dt, a = want[t.Name]
        assert tuple(t.Shape) == tuple(ne)
        assert t.TypeSize == (2 if dt == "f16" else 4)
        assert np.array_equal(t.to_numpy(), a)
    # widened chunks are the float32 values of the halves, as the reference's GetDataRaw yields them
    q = next(t for t in tensors if t.Name == "blk.0.attn_q.weight")
    wide = np.frombuffer(b"".join(q.get_data_raw(widen_half=True)), np.float32)
    assert np.array_equal(wide, want[q.Name][2].astype(np.float32).reshape(-1))


# ---- the native GGUF directory reader on files it must refuse (no device involved) ------------------------------
def _probe(path, ctx=64):
    import ctypes as C

    from nfai_b200 import _lib
    lib = _lib.load()
    hp = _lib.HParams()
    err = C.create_string_buffer(256)
    rc = lib.nfai_gguf_probe(str(path).encode(), ctx, C.byref(hp), err, len(err))
    return rc, hp, err.value.decode()


def _gguf_bytes(tmp_path):
    cfg = synth.get_config("s3")
    path = os.path.join(tmp_path, "ok.gguf")
    gguf_io.write_synthetic_gguf(cfg, path, seed=3)
    return cfg, path, bytearray(open(path, "rb").read())


def test_gguf_probe_reads_the_geometry(tmp_path):
    cfg, path, _ = _gguf_bytes(tmp_path)
    rc, hp, err = _probe(path)
    assert rc == 0, err
    assert (hp.H, hp.L, hp.qH, hp.kvH, hp.d, hp.F, hp.V) == (cfg.H, cfg.L, cfg.qH, cfg.kvH, cfg.d, cfg.F, cfg.V)
    assert hp.ctx == 64 and hp.tied == (1 if cfg.tied else 0)


def test_gguf_probe_refuses_truncated_files(tmp_path):
    _, _, data = _gguf_bytes(tmp_path)
    from nfai_b200 import _lib
    for keep in (8, 23, 24, 40, 200, len(data) // 2, len(data) - 1):
        p = os.path.join(tmp_path, f"cut{keep}.gguf")
        open(p, "wb").write(data[:keep])
        rc, _, err = _probe(p)
        assert rc == _lib.ERR_ARG and err, (keep, rc, err)


def test_gguf_probe_refuses_hostile_headers(tmp_path):
    import struct

    from nfai_b200 import _lib
    _, _, data = _gguf_bytes(tmp_path)

    def variant(name, edit):
        d = bytearray(data)
        edit(d)
        p = os.path.join(tmp_path, name)
        open(p, "wb").write(d)
        rc, _, err = _probe(p)
        assert rc == _lib.ERR_ARG and err, (name, rc, err)
        return err

    # counts that cannot be true
    variant("kv.gguf", lambda d: d.__setitem__(slice(16, 24), struct.pack("<Q", 1 << 62)))
    variant("nt.gguf", lambda d: d.__setitem__(slice(8, 16), struct.pack("<Q", 0xFFFFFFFFFFFFFFFF)))
    # a key length that wraps off + len
    variant("key.gguf", lambda d: d.__setitem__(slice(24, 32), struct.pack("<Q", 0xFFFFFFFFFFFFFFF0)))
    # an array whose element count times element size wraps
    def big_array(d):
        i = d.find(b"tokenizer.ggml.tokens")
        if i < 0:
            i = d.find(b"general.architecture")
        key_end = i + len(b"general.architecture") if d[i:i + 7] == b"general" else i + len(b"tokenizer.ggml.tokens")
        d[key_end:key_end + 16] = struct.pack("<IIQ", 9, 10, 0x2000000000000001)  # array of u64, count * 8 wraps
    variant("arr.gguf", big_array)

    def set_alignment(value):
        def edit(d):
            i = d.find(b"general.alignment")
            assert i > 0
            d[i + 17 + 4:i + 17 + 8] = struct.pack("<I", value)
        return edit
    assert "alignment" in variant("a0.gguf", set_alignment(0))
    assert "alignment" in variant("a3.gguf", set_alignment(3))

    def far_tensor(d):
        i = d.find(b"blk.0.ffn_down.weight")
        assert i > 0
        off = i + len(b"blk.0.ffn_down.weight") + 4 + 16 + 4  # n_dims, two dims, type
        d[off:off + 8] = struct.pack("<Q", 0xFFFFFFFFFFFFFF00)
    assert "beyond" in variant("far.gguf", far_tensor)

    def huge_dim(d):
        i = d.find(b"blk.0.ffn_down.weight")
        off = i + len(b"blk.0.ffn_down.weight") + 4
        d[off:off + 8] = struct.pack("<Q", 1 << 63)
    variant("dim.gguf", huge_dim)
