"""GGUF reader against files written by gguf.GGUFWriter -- the writer the reference's converters use
(scripts/gguf_common.py:40-52: F32 tensors as float32 arrays, BF16 tensors as uint16 bit patterns with
raw_dtype BF16; metadata through add_uint32 / add_float32 / add_float64 / add_string / add_bool).  Host only."""
import numpy as np
import pytest

gguf = pytest.importorskip("gguf")

from oracle import oracle_ffi as orc


def _write(path, arch="pi0"):
    rng = np.random.default_rng(7)
    w = gguf.GGUFWriter(str(path), arch)
    w.add_uint32("pi0.hidden", 2048)
    w.add_uint32("pi0.n_layers", 3)
    w.add_float32("pi0.rms_norm_eps", 1e-6)
    w.add_float64("pi0.min_period", 4e-3)
    w.add_string("pi0.paligemma_variant", "gemma_2b")
    w.add_bool("pi0.use_adarms_expert", True)
    w.add_array("pi0.some_list", [1, 2, 3])
    w.add_array("pi0.some_names", ["a", "bc"])
    t = {}
    t["a.f32"] = rng.standard_normal((5, 24)).astype(np.float32)
    w.add_tensor("a.f32", t["a.f32"], raw_dtype=gguf.GGMLQuantizationType.F32)
    bf = orc.bf16_round(rng.standard_normal((7, 16)).astype(np.float32))
    t["b.bf16"] = bf
    w.add_tensor("b.bf16", orc.f32_to_bf16_bits(bf).astype(np.uint16), raw_shape=[7, 16],
                 raw_dtype=gguf.GGMLQuantizationType.BF16)
    t["c.f16"] = rng.standard_normal((3, 8)).astype(np.float16)
    t["c.f16"][0, 0] = np.float16(6e-8)  # subnormal half
    w.add_tensor("c.f16", t["c.f16"])
    t["d.vec"] = rng.standard_normal(33).astype(np.float32)
    w.add_tensor("d.vec", t["d.vec"])
    t["e.i8"] = rng.integers(-128, 127, (4, 32), dtype=np.int8)
    w.add_tensor("e.i8", t["e.i8"], raw_dtype=gguf.GGMLQuantizationType.I8)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()
    return t


def test_reads_what_the_reference_writer_wrote(tmp_path):
    import vla_cpp_b200 as vb

    path = tmp_path / "m.gguf"
    t = _write(path)
    g = vb.Gguf(path)
    assert g.names() == ["a.f32", "b.bf16", "c.f16", "d.vec", "e.i8"]
    assert g.meta("general.architecture") == "pi0"
    assert g.meta("pi0.hidden") == 2048 and g.meta("pi0.n_layers") == 3
    assert g.meta("pi0.rms_norm_eps") == pytest.approx(1e-6) and g.meta("pi0.min_period") == 4e-3
    assert g.meta("pi0.paligemma_variant") == "gemma_2b"
    assert g.meta("pi0.absent") is None and g.meta("pi0.some_list") is None
    assert g.info("a.f32") == (0, [24, 5], 5 * 24 * 4)      # dims fastest-first, like ggml's ne[]
    assert g.info("b.bf16") == (30, [16, 7], 7 * 16 * 2)
    assert g.info("c.f16") == (1, [8, 3], 3 * 8 * 2)
    assert g.info("d.vec") == (0, [33], 33 * 4)
    assert g.info("e.i8") == (24, [32, 4], 4 * 32)
    assert g.info("nope") is None
    assert np.array_equal(g.f32("a.f32"), t["a.f32"])
    assert np.array_equal(g.f32("b.bf16"), t["b.bf16"])
    assert np.array_equal(g.f32("c.f16"), t["c.f16"].astype(np.float32))
    assert np.array_equal(g.f32("d.vec", gemma_norm=True), t["d.vec"] + np.float32(1.0))
    assert np.array_equal(g.raw("e.i8").view(np.int8).reshape(4, 32), t["e.i8"])
    with pytest.raises(vb.VlaB200Error):
        g.f32("e.i8")  # not a float type
    g.close()


def test_rejects_damaged_files(tmp_path):
    import vla_cpp_b200 as vb

    path = tmp_path / "m.gguf"
    _write(path)
    data = path.read_bytes()
    (tmp_path / "magic.gguf").write_bytes(b"GGML" + data[4:])
    (tmp_path / "short.gguf").write_bytes(data[: len(data) - 64])   # last tensor runs past the end
    (tmp_path / "dir.gguf").write_bytes(data[:200])                 # cut inside the metadata
    for name in ("magic.gguf", "short.gguf", "dir.gguf", "missing.gguf"):
        with pytest.raises(vb.VlaB200Error):
            vb.Gguf(tmp_path / name)


def test_truncations_and_corrupt_directories_never_crash(tmp_path):
    """Every read of the parser is bounds-checked: a file cut anywhere, or with bytes of its header / directory
    overwritten, either opens (and then every listed tensor lies inside the file) or is refused."""
    import vla_cpp_b200 as vb

    path = tmp_path / "m.gguf"
    _write(path)
    data = path.read_bytes()
    rng = np.random.default_rng(3)
    cases = [data[:n] for n in list(range(0, 64, 7)) + [int(x) for x in rng.integers(64, len(data), 40)]]
    for _ in range(60):  # corrupt a few bytes in the first 1.5 KB (header, metadata, tensor directory)
        b = bytearray(data)
        for pos in rng.integers(4, min(1536, len(data)), 3):
            b[int(pos)] = int(rng.integers(0, 256))
        cases.append(bytes(b))
    opened = 0
    for i, blob in enumerate(cases):
        p = tmp_path / f"case{i}.gguf"
        p.write_bytes(blob)
        try:
            g = vb.Gguf(p)
        except vb.VlaB200Error:
            continue
        opened += 1
        for name in g.names():
            inf = g.info(name)
            assert inf is not None
            if inf[2]:
                assert len(g.raw(name)) == inf[2]  # readable end to end: lies inside the mapping
        g.close()
    assert opened < len(cases)
