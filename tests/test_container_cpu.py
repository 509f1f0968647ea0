"""The ``.bin`` container reader and writer against a file written by the reference's own Python tools
(tests/golden/container_small.bin, made by tests/golden/make_container_fixture.py), and the loader conventions
built on it (``_scale`` / ``_smooth_inv`` / ``_act_scale``, group size from the scale's shape)."""
import struct
from pathlib import Path

import numpy as np
import pytest

from fish_audio_cpp_b200 import container as ct

GOLDEN = Path(__file__).resolve().parent / "golden"
P0 = "text_model.model.layers.0."


@pytest.fixture(scope="module")
def golden():
    return ct.Container(GOLDEN / "container_small.bin"), np.load(GOLDEN / "container_small_expected.npz")


def test_reads_what_the_reference_wrote(golden):
    c, want = golden
    assert c.names() == list(want.files)  # file order
    for name in want.files:
        got = c.get(name)
        assert got.dtype == want[name].dtype and got.shape == want[name].shape, name
        assert np.array_equal(got.view(np.uint8), want[name].view(np.uint8)), name
        assert c.entries[name].data_offset % 256 == 0
    assert c.data_section_offset == 12 + 344 * len(want.files)


def test_writer_is_byte_identical_to_the_reference_writer(golden, tmp_path):
    c, want = golden
    out = tmp_path / "rewritten.bin"
    ct.write_container(out, {n: want[n] for n in want.files})
    assert out.read_bytes() == (GOLDEN / "container_small.bin").read_bytes()


def test_loader_conventions(golden):
    c, _ = golden
    assert sorted(c.w8a8_linears()) == sorted(P0 + n for n in ["attention.wqkv.weight", "attention.wo.weight",
                                                               "feed_forward.w1.weight", "feed_forward.w3.weight",
                                                               "feed_forward.w2.weight"])
    assert not c.is_w8a8(P0 + "attention_norm.weight")
    # group size as infer_group_size_from_scale: K for a 1-D scale, else ceil(K / groups)
    assert c.group_size(P0 + "attention.wqkv.weight") == 256
    assert c.group_size(P0 + "attention.wo.weight") == 64
    assert c.group_size(P0 + "feed_forward.w2.weight") == 300
    w1 = c.linear(P0 + "feed_forward.w1.weight")
    assert (w1.N, w1.K, w1.G, w1.group_size) == (32, 512, 2, 256)
    assert w1.smooth_inv is not None and w1.smooth_inv.shape == (512,) and w1.act_scale is None
    assert c.linear(P0 + "attention.wo.weight").smooth_inv is None
    w2 = c.linear(P0 + "feed_forward.w2.weight")
    assert w2.scale.shape == (16,) and w2.G == 1
    with pytest.raises(KeyError, match="Tensor not found"):
        c.get("nope")
    with pytest.raises(KeyError):
        c.linear(P0 + "attention_norm.weight")


def test_the_reference_quantiser_gives_codes_our_scales_reproduce(golden):
    """The exporter's weight codes are round(w / scale) clipped to +-127 (tools/quant_utils.py:171-194): every code
    is within the range and every row of a group reaches 127 in magnitude (the scale is the row's absmax / 127)."""
    c, _ = golden
    lin = c.linear(P0 + "attention.wo.weight")
    assert np.abs(lin.W.astype(np.int32)).max() == 127
    per_group = np.abs(lin.W.astype(np.int32)).reshape(lin.N, lin.G, lin.group_size).max(axis=2)
    assert (per_group >= 126).all()  # fp16 rounding of the scale may cost one step
    assert (lin.scale.astype(np.float32) > 0).all()


def test_gate_up_fuse_only_with_one_smooth_vector(golden, tmp_path):
    c, want = golden
    assert list(ct.fused_gate_up_names(c)) == [(P0 + "feed_forward.", P0 + "feed_forward.w1.weight", P0 + "feed_forward.w3.weight")]
    tensors = {n: np.array(want[n]) for n in want.files}
    tensors[P0 + "feed_forward.w3.weight_smooth_inv"][5] = np.float16(3.0)
    ct.write_container(tmp_path / "two_vectors.bin", tensors)
    assert list(ct.fused_gate_up_names(ct.Container(tmp_path / "two_vectors.bin"))) == []
    del tensors[P0 + "feed_forward.w3.weight_smooth_inv"]
    ct.write_container(tmp_path / "one_side.bin", tensors)
    assert list(ct.fused_gate_up_names(ct.Container(tmp_path / "one_side.bin"))) == []


def _patched(tmp_path, name, offset, payload):
    raw = bytearray((GOLDEN / "container_small.bin").read_bytes())
    raw[offset: offset + len(payload)] = payload
    p = tmp_path / name
    p.write_bytes(bytes(raw))
    return p


def test_refuses_what_the_reference_loader_refuses(tmp_path):
    with pytest.raises(ct.ContainerError, match="invalid magic"):
        ct.Container(_patched(tmp_path, "magic.bin", 0, struct.pack("<I", 0x12345678)))
    with pytest.raises(ct.ContainerError, match="unsupported version"):
        ct.Container(_patched(tmp_path, "version.bin", 4, struct.pack("<I", 2)))
    short = tmp_path / "short.bin"
    short.write_bytes((GOLDEN / "container_small.bin").read_bytes()[:100])
    with pytest.raises(ct.ContainerError, match="do not fit"):
        ct.Container(short)
    tiny = tmp_path / "tiny.bin"
    tiny.write_bytes(b"FISH")
    with pytest.raises(ct.ContainerError, match="preamble"):
        ct.Container(tiny)


def test_refuses_headers_that_point_outside_the_file(tmp_path):
    first = 12  # header 0: name[256] dtype ndim shape[8] offset size
    with pytest.raises(ct.ContainerError, match="outside the file"):
        ct.Container(_patched(tmp_path, "offset.bin", first + 256 + 8 + 64, struct.pack("<Q", 1 << 40)))
    with pytest.raises(ct.ContainerError, match="unaligned"):
        ct.Container(_patched(tmp_path, "unaligned.bin", first + 256 + 8 + 64, struct.pack("<Q", 5121)))
    with pytest.raises(ct.ContainerError, match="bytes for shape"):
        ct.Container(_patched(tmp_path, "size.bin", first + 256 + 8 + 64 + 8, struct.pack("<Q", 3)))
    with pytest.raises(ct.ContainerError, match="unknown dtype"):
        ct.Container(_patched(tmp_path, "dtype.bin", first + 256, struct.pack("<I", 9)))
    with pytest.raises(ct.ContainerError, match="dimensions"):
        ct.Container(_patched(tmp_path, "ndim.bin", first + 256 + 4, struct.pack("<I", 9)))


def test_writer_limits(tmp_path):
    with pytest.raises(ct.ContainerError, match="too long"):
        ct.write_container(tmp_path / "a.bin", {"x" * 256: np.zeros(1, np.float32)})
    with pytest.raises(ct.ContainerError, match="no container code"):
        ct.write_container(tmp_path / "b.bin", {"x": np.zeros(1, np.float64)})
    ct.write_container(tmp_path / "c.bin", {"bf": np.arange(4, dtype=np.uint16)}, {"bf": ct.DTYPE_BF16})
    c = ct.Container(tmp_path / "c.bin")
    assert c.entries["bf"].dtype_val == ct.DTYPE_BF16 and c.get("bf").tolist() == [0, 1, 2, 3]
    ct.write_container(tmp_path / "empty.bin", {})
    assert ct.Container(tmp_path / "empty.bin").names() == []


# ---------------------------------------------------------------- the library's native reader (include/w8a8_container.h)
@pytest.fixture(scope="module")
def native(pkg):
    from fish_audio_cpp_b200 import capi

    c = capi.NativeContainer(GOLDEN / "container_small.bin")
    yield c
    c.close()


def test_native_reader_sees_what_the_reference_wrote(native, golden):
    """The C ABI reader over the file the reference's tools wrote: same tensors in the same order, same element
    types, shapes, offsets and bytes as the Python reader and as the arrays the fixture was made from."""
    c, want = golden
    assert len(native) == len(want.files) and native.data_section_offset == 12 + 344 * len(want.files)
    codes = {np.dtype("<f4"): 0, np.dtype("<f2"): 1, np.dtype("i1"): 3}
    for i, name in enumerate(want.files):
        info = native.tensor(i)
        assert info.name.decode() == name and native.find(name) == i
        assert info.dtype == codes[want[name].dtype] and info.ndim == want[name].ndim
        assert tuple(info.shape[:info.ndim]) == want[name].shape and not any(info.shape[info.ndim:8])
        e = c.entries[name]
        assert (info.offset, info.nbytes) == (e.data_offset, e.data_size) and info.offset % 256 == 0
        assert native.bytes_of(i) == want[name].tobytes()
    assert native.find("nope") == -1


def test_native_reader_loader_conventions(native, golden, pkg):
    c, _ = golden
    for name in c.w8a8_linears():  # infer_group_size_from_scale, dual_ar_engine.cc:17-24
        assert native.group_size(name) == c.group_size(name), name
    assert native.group_size(P0 + "feed_forward.w2.weight") == 300 and native.group_size(P0 + "attention.wo.weight") == 64
    with pytest.raises(pkg.W8A8Error, match="not an int8 tensor with a _scale"):
        native.group_size(P0 + "attention_norm.weight")
    with pytest.raises(pkg.W8A8Error, match="Tensor not found"):
        native.group_size("nope")
    with pytest.raises(pkg.W8A8Error):
        native.tensor(len(native))


def test_native_reader_refuses_what_the_python_reader_refuses(tmp_path, pkg):
    from fish_audio_cpp_b200 import capi

    first = 12
    cases = [("magic.bin", 0, struct.pack("<I", 0x12345678), "Invalid magic: 0x12345678, expected 0x46495348"),
             ("version.bin", 4, struct.pack("<I", 2), "Unsupported version: 2"),
             ("offset.bin", first + 256 + 8 + 64, struct.pack("<Q", 1 << 40), "outside the file"),
             ("unaligned.bin", first + 256 + 8 + 64, struct.pack("<Q", 5121), "unaligned"),
             ("size.bin", first + 256 + 8 + 64 + 8, struct.pack("<Q", 3), "do not match its shape"),
             ("dtype.bin", first + 256, struct.pack("<I", 9), "unknown dtype 9"),
             ("ndim.bin", first + 256 + 4, struct.pack("<I", 9), "9 dimensions"),
             ("negative.bin", first + 256 + 8, struct.pack("<q", -4), "negative extent"),
             ("huge.bin", first + 256 + 8, struct.pack("<q", 1 << 62), "overflow|do not match")]
    for fname, at, patch, msg in cases:
        with pytest.raises(pkg.W8A8Error, match=msg) as e:
            capi.NativeContainer(_patched(tmp_path, fname, at, patch))
        assert e.value.status == 1  # W8A8_ERR_INVALID_ARG
    short = tmp_path / "short.bin"
    short.write_bytes((GOLDEN / "container_small.bin").read_bytes()[:100])
    with pytest.raises(pkg.W8A8Error, match="do not fit"):
        capi.NativeContainer(short)
    tiny = tmp_path / "tiny.bin"
    tiny.write_bytes(b"FISH")
    with pytest.raises(pkg.W8A8Error, match="preamble"):
        capi.NativeContainer(tiny)
    with pytest.raises(pkg.W8A8Error, match="Failed to open model file"):
        capi.NativeContainer(tmp_path / "missing.bin")


def test_native_reader_reads_a_sidecar_written_in_the_same_format(tmp_path, pkg):
    """What write_container writes (the packed sidecar uses it) is a file the native reader takes: uint8 images come
    back as int8 tensors of the same bytes, names of up to 255 bytes survive."""
    from fish_audio_cpp_b200 import capi

    rng = np.random.default_rng(1)
    tensors = {"a" * 255: rng.integers(0, 256, (3, 5), dtype=np.uint8), "w_packed_meta": np.array([16, 256, 64], np.float32),
               "h": rng.standard_normal((2, 3, 4)).astype(np.float16)}
    path = tmp_path / "sidecar.bin"
    ct.write_container(path, tensors)
    c = capi.NativeContainer(path)
    try:
        assert len(c) == 3
        for i, (name, arr) in enumerate(tensors.items()):
            info = c.tensor(i)
            assert info.name.decode() == name and tuple(info.shape[:info.ndim]) == arr.shape
            assert c.bytes_of(i) == arr.tobytes()
        assert c.tensor(0).dtype == 3
    finally:
        c.close()


def test_native_reader_pin_without_a_device_is_an_error_not_a_crash(native, pkg):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present: pinning would succeed")
    with pytest.raises(pkg.W8A8Error) as e:
        native.pin()
    assert e.value.status == 3  # W8A8_ERR_CUDA
