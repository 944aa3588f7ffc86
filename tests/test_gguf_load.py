"""The model-file side: the GGUF reader against the writer's own bookkeeping and against the reference's
reader (where oracle/_ref is built), malformed files, and loading a file into the graph driver: logits of a
model loaded from a file equal those of the same bytes handed over tensor by tensor."""
import struct

import numpy as np
import pytest

TINY = dict(n_layer=2, n_embd=256, n_head=4, n_head_kv=2, n_ff=512, n_vocab=512, rope_theta=500000.0, rms_eps=1e-5)


@pytest.fixture(scope="module")
def tiny_gguf(b200, tmp_path_factory):
    from llama_cpp_b200 import gguf_synth
    path = tmp_path_factory.mktemp("gguf") / "tiny.gguf"
    n = gguf_synth.write_llama_gguf(path, TINY, seed_base=500)
    assert path.stat().st_size == n
    return path


def _s(x):
    b = x.encode()
    return struct.pack("<Q", len(b)) + b


def test_reader_matches_writer(b200, tiny_gguf):
    from llama_cpp_b200 import gguf, gguf_synth
    with gguf.GGUF(tiny_gguf) as g:
        assert g.version == 3 and g.alignment == 32 and g.data_offset % 32 == 0
        assert g.get_str("general.architecture") == "llama"
        assert g.get_u32("llama.block_count") == TINY["n_layer"]
        assert g.get_u32("llama.attention.head_count_kv") == TINY["n_head_kv"]
        assert abs(g.get_f32("llama.rope.freq_base") - 500000.0) < 1e-3
        assert g.get_u32("no.such.key") is None and g.get_str("llama.block_count") is None
        want = gguf_synth.tensor_list(TINY)
        got = g.tensors()
        assert [t["name"] for t in got] == [w[0] for w in want]
        off = 0
        for t, (name, ty, ne0, ne1) in zip(got, want):
            assert t["type"] == ty and t["ne"][0] == ne0 and t["ne"][1] == ne1 and t["offset"] == off
            assert t["nbytes"] == gguf_synth.row_bytes(ty, ne0) * ne1
            off += (t["nbytes"] + 31) // 32 * 32
        assert g.find("blk.1.ffn_down.weight") == got[-1]["index"] and g.find("nope") == -1
        # the bytes of a tensor are the bytes the writer's generator produces for it
        from llama_cpp_b200 import synth
        i = g.find("blk.0.attn_q.weight")
        name, ty, ne0, ne1 = want[i]
        assert np.array_equal(g.tensor_bytes(i, got[i]["nbytes"]), synth.make_tensor(ty, ne0, ne1, seed=500 + i))


def test_reader_matches_reference_reader(b200, oracle, tiny_gguf, tmp_path):
    if not oracle.ref_available():
        pytest.skip("reference build (oracle/_ref) not present")
    from llama_cpp_b200 import gguf
    # a second file with every value type, arrays of scalars and of strings, and a non-default alignment
    kvs = [(_s("general.alignment") + struct.pack("<II", 4, 64)),
           (_s("a.u8") + struct.pack("<IB", 0, 7)), (_s("a.i8") + struct.pack("<Ib", 1, -7)),
           (_s("a.u16") + struct.pack("<IH", 2, 600)), (_s("a.i16") + struct.pack("<Ih", 3, -600)),
           (_s("a.i32") + struct.pack("<Ii", 5, -70000)), (_s("a.f32") + struct.pack("<If", 6, 1.5)),
           (_s("a.bool") + struct.pack("<IB", 7, 1)), (_s("a.str") + struct.pack("<I", 8) + _s("hello")),
           (_s("a.arr_i32") + struct.pack("<IIQ", 9, 5, 3) + struct.pack("<3i", 1, 2, 3)),
           (_s("a.arr_str") + struct.pack("<IIQ", 9, 8, 2) + _s("x") + _s("yz")),
           (_s("a.u64") + struct.pack("<IQ", 10, 1 << 40)), (_s("a.i64") + struct.pack("<Iq", 11, -5)),
           (_s("a.f64") + struct.pack("<Id", 12, 2.25))]
    infos = [_s("t0") + struct.pack("<IQQIQ", 2, 32, 3, 2, 0),            # Q4_0 [32, 3]: 54 bytes -> next at 64
             _s("t1") + struct.pack("<IQIQ", 1, 5, 0, 64)]                # F32 [5]
    head = b"GGUF" + struct.pack("<IQQ", 3, len(infos), len(kvs)) + b"".join(kvs) + b"".join(infos)
    head += b"\0" * (-len(head) % 64)
    p2 = tmp_path / "mixed.gguf"
    p2.write_bytes(head + bytes(range(54)) + b"\0" * 10 + struct.pack("<5f", 1, 2, 3, 4, 5))
    for path in (tiny_gguf, p2):
        ref = oracle.ref_gguf_directory(path)
        assert ref is not None
        with gguf.GGUF(path) as g:
            assert (g.version, g.alignment, g.data_offset) == (ref["version"], ref["alignment"], ref["data_offset"])
            assert [(k, t) for k, t, _, _ in g.keys()] == ref["keys"]
            mine = g.tensors()
            assert [(t["name"], t["type"], t["offset"], t["nbytes"]) for t in mine] == \
                   [(t["name"], t["type"], t["offset"], t["nbytes"]) for t in ref["tensors"]]
    with gguf.GGUF(p2) as g:
        assert g.get_u32("a.u8") == 7 and g.get_u32("a.i8") is None and g.get_f32("a.f64") == 2.25
        assert g.get_str("a.str") == "hello"
        assert dict((k, (et, n)) for k, t, et, n in g.keys() if t == 9) == {"a.arr_i32": (5, 3), "a.arr_str": (8, 2)}
        assert np.array_equal(g.tensor_bytes(1, 20).view(np.float32), np.arange(1, 6, dtype=np.float32))


def test_reader_rejects_malformed_files(b200, tiny_gguf, tmp_path):
    from llama_cpp_b200 import gguf
    raw = tiny_gguf.read_bytes()
    cases = {
        "magic": b"GGML" + raw[4:],
        "version": raw[:4] + struct.pack("<I", 1) + raw[8:],
        "counts": raw[:8] + struct.pack("<QQ", 1 << 60, 1 << 60) + raw[24:],
        "short": raw[:20],
        "truncated_meta": raw[:200],
        "truncated_data": raw[:len(raw) - 4096],
        "string_length": raw[:24] + struct.pack("<Q", 1 << 50) + raw[32:],
    }
    for name, data in cases.items():
        p = tmp_path / f"{name}.gguf"
        p.write_bytes(data)
        with pytest.raises(b200.B200Error):
            gguf.GGUF(p)
    with pytest.raises(b200.B200Error):
        gguf.GGUF(tmp_path / "does_not_exist.gguf")


def _from_tensors(b200, reg, path, arch=TINY):
    """The same model built tensor by tensor from the file's bytes."""
    from llama_cpp_b200 import gguf, llama
    m = llama.Llama(n_ctx=512, n_ubatch=64, reg=reg, n_threads=2, **arch)
    with gguf.GGUF(path) as g:
        for t in m.tensors():
            i = g.find(t["name"])
            info = g.tensors()[i]
            rows = g.tensor_bytes(i, info["nbytes"]).reshape(t["full_rows"], -1)
            m.set_tensor(t["index"], rows[t["row_low"]:t["row_low"] + t["ne1"]])
    return m


def _logits(m):
    toks = np.random.default_rng(1).integers(0, m.cfg.n_vocab, 21).astype(np.int32)
    return [m.decode(toks[:20], 0).copy(), m.decode(toks[20:], 20).copy()]



@pytest.mark.parametrize("weight_type,file_type", [(2, 2), (8, 7)])           # Q4_0, Q8_0
def test_single_type_files(b200, oracle, tmp_path, weight_type, file_type):
    """Files with every matrix in one simple type (what `llama-quantize ... Q4_0 / Q8_0` leaves, output.weight in Q6_K for
    Q4_0): types and sizes as the reader sees them, and the model loads and decodes on the reference CPU backend with the
    logits of the same weights stored as F32 (the blocks' decoded values) within the activation-quantization error."""
    from llama_cpp_b200 import gguf, gguf_synth, llama
    path = tmp_path / "m.gguf"
    gguf_synth.write_llama_gguf(path, TINY, seed_base=90, weight_type=weight_type)
    with gguf.GGUF(path) as g:
        assert g.get_u32("general.file_type") == file_type
        for t in g.tensors():
            one_d = len(t["ne"]) < 2 or t["ne"][1] == 1
            want = 0 if one_d else (14 if (t["name"] == "output.weight" and weight_type == 2) else weight_type)
            assert t["type"] == want, t
            assert t["nbytes"] == gguf_synth.row_bytes(want, t["ne"][0]) * (1 if one_d else t["ne"][1])
    if not oracle.ref_available():
        pytest.skip("reference build (oracle/_ref) not present")
    reg = oracle.ref_cpu_backend_reg()
    names = {0: "f32", 2: "q4_0", 8: "q8_0", 14: "q6_K"}
    exact = tmp_path / "exact.gguf"
    gguf_synth.write_llama_gguf(exact, TINY, seed_base=90, weight_type=weight_type,
                                dequantize=lambda ty, raw, ne0: oracle.dequantize_rows(names[ty], np.asarray(raw).reshape(-1, gguf_synth.row_bytes(ty, ne0)), ne0))
    a = llama.Llama.from_gguf(path, n_ctx=512, n_ubatch=64, reg=reg, n_threads=2)
    b = llama.Llama.from_gguf(exact, n_ctx=512, n_ubatch=64, reg=reg, n_threads=2)
    try:
        for x, y in zip(_logits(a), _logits(b)):
            assert np.isfinite(x).all() and oracle.nmse(y, x) < 2e-3
    finally:
        a.close(); b.close()


def test_load_into_driver_on_reference_cpu_backend(b200, oracle, tiny_gguf):
    if not oracle.ref_available():
        pytest.skip("reference build (oracle/_ref) not present")
    from llama_cpp_b200 import llama
    reg = oracle.ref_cpu_backend_reg()
    a = llama.Llama.from_gguf(tiny_gguf, n_ctx=512, n_ubatch=64, reg=reg, n_threads=2)
    b = _from_tensors(b200, reg, tiny_gguf)
    try:
        for k in ("n_layer", "n_embd", "n_head", "n_head_kv", "n_ff", "n_vocab"):
            assert getattr(a.cfg, k) == TINY[k]
        assert abs(a.cfg.rope_theta - 500000.0) < 1e-3 and abs(a.cfg.rms_eps - 1e-5) < 1e-9
        assert [(t["name"], t["type"], t["ne0"], t["ne1"]) for t in a.tensors()] == [(t["name"], t["type"], t["ne0"], t["ne1"]) for t in b.tensors()]
        for x, y in zip(_logits(a), _logits(b)):
            assert np.array_equal(x.view(np.uint32), y.view(np.uint32))
    finally:
        a.close(); b.close()


def test_rope_frequency_factors_from_file(b200, oracle, tiny_gguf, tmp_path):
    """rope_freqs.weight becomes the third operand of every ROPE: factors of one change nothing (bit for bit),
    other factors change the logits."""
    if not oracle.ref_available():
        pytest.skip("reference build (oracle/_ref) not present")
    from llama_cpp_b200 import gguf_synth, llama
    reg = oracle.ref_cpu_backend_reg()
    hd2 = TINY["n_embd"] // TINY["n_head"] // 2
    ones, ramp = tmp_path / "ones.gguf", tmp_path / "ramp.gguf"
    gguf_synth.write_llama_gguf(ones, TINY, seed_base=500, rope_freqs=np.ones(hd2, np.float32))
    gguf_synth.write_llama_gguf(ramp, TINY, seed_base=500, rope_freqs=np.linspace(1.0, 8.0, hd2).astype(np.float32))
    outs = []
    for p in (tiny_gguf, ones, ramp):
        m = llama.Llama.from_gguf(p, n_ctx=512, n_ubatch=64, reg=reg, n_threads=2)
        assert [t["name"] for t in m.tensors()][-1] == ("blk.1.ffn_down.weight" if p == tiny_gguf else "rope_freqs.weight")
        outs.append(_logits(m))
        m.close()
    for x, y in zip(outs[0], outs[1]):
        assert np.array_equal(x.view(np.uint32), y.view(np.uint32))
    assert oracle.nmse(outs[0][1], outs[2][1]) > 1e-6


def test_load_rejects_unsupported_models(b200, oracle, tiny_gguf, tmp_path):
    from llama_cpp_b200 import llama
    raw = tiny_gguf.read_bytes()
    bad = tmp_path / "arch.gguf"
    bad.write_bytes(raw.replace(_s("general.architecture") + struct.pack("<I", 8) + _s("llama"),
                                _s("general.architecture") + struct.pack("<I", 8) + _s("gpt2x"), 1))
    with pytest.raises(b200.B200Error, match="not llama"):
        llama.Llama.from_gguf(bad, n_ctx=512, n_ubatch=64)
    with pytest.raises(b200.B200Error):
        llama.Llama.from_gguf(tmp_path / "missing.gguf", n_ctx=512, n_ubatch=64)
    # hyper-parameters a corrupt file may carry: an error, never a division by zero or a wild allocation
    if oracle.ref_available():
        reg = oracle.ref_cpu_backend_reg()
        for key, value in (("llama.attention.head_count_kv", 0), ("llama.block_count", 0), ("llama.embedding_length", 0),
                           ("llama.feed_forward_length", 0x7fffff00)):
            i = raw.index(_s(key) + struct.pack("<I", 4))
            at = i + len(_s(key)) + 4
            broken = tmp_path / "hp.gguf"
            broken.write_bytes(raw[:at] + struct.pack("<I", value) + raw[at + 4:])
            with pytest.raises(b200.B200Error):
                llama.Llama.from_gguf(broken, n_ctx=512, n_ubatch=64, reg=reg)
        with pytest.raises(b200.B200Error):
            llama.Llama.from_gguf(tiny_gguf, n_ctx=0, n_ubatch=64, reg=reg)


@pytest.mark.gpu
def test_load_into_driver_on_b200(b200, tiny_gguf):
    from llama_cpp_b200 import llama
    a = llama.Llama.from_gguf(tiny_gguf, n_ctx=512, n_ubatch=64)
    b = _from_tensors(b200, None, tiny_gguf)
    try:
        for x, y in zip(_logits(a), _logits(b)):
            assert np.isfinite(x).all() and np.array_equal(x.view(np.uint32), y.view(np.uint32))
        assert a.launch_count > 0
    finally:
        a.close(); b.close()


@pytest.mark.gpu
def test_rope_frequency_factors_b200_matches_reference_cpu_backend(b200, oracle, tmp_path):
    if not oracle.ref_available():
        pytest.skip("reference build (oracle/_ref) not present")
    from llama_cpp_b200 import gguf_synth, llama
    arch = dict(n_layer=2, n_embd=1024, n_head=8, n_head_kv=2, n_ff=2048, n_vocab=2048, rope_theta=500000.0, rms_eps=1e-5)
    path = tmp_path / "ff.gguf"
    gguf_synth.write_llama_gguf(path, arch, seed_base=40, rope_freqs=np.linspace(1.0, 8.0, 64).astype(np.float32))
    cpu = llama.Llama.from_gguf(path, n_ctx=512, n_ubatch=64, reg=oracle.ref_cpu_backend_reg(), n_threads=8)
    gpu = llama.Llama.from_gguf(path, n_ctx=512, n_ubatch=64)
    try:
        for x, y in zip(_logits(cpu), _logits(gpu)):
            assert oracle.nmse(x, y) <= 5e-4 * (7 * arch["n_layer"] + 1)       # per-op criterion x chained MUL_MATs
    finally:
        cpu.close(); gpu.close()


@pytest.mark.gpu
def test_load_large_tensor_through_staging(b200, tmp_path):
    """Tensors of several staging chunks (and not a multiple of the chunk size), spread over the upload workers, arrive intact: the loaded model's
    logits equal those of the tensor-by-tensor model."""
    from llama_cpp_b200 import gguf_synth, llama
    arch = dict(n_layer=1, n_embd=1024, n_head=8, n_head_kv=2, n_ff=2048, n_vocab=70016, rope_theta=10000.0, rms_eps=1e-6)
    path = tmp_path / "wide.gguf"
    gguf_synth.write_llama_gguf(path, arch, seed_base=9, device="cuda")
    a = llama.Llama.from_gguf(path, n_ctx=512, n_ubatch=64)
    b = _from_tensors(b200, None, path, arch)
    try:
        assert abs(a.cfg.rms_eps - 1e-6) < 1e-12 and a.cfg.n_vocab == 70016
        for x, y in zip(_logits(a), _logits(b)):
            assert np.array_equal(x.view(np.uint32), y.view(np.uint32))
    finally:
        a.close(); b.close()
