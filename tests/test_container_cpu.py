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
