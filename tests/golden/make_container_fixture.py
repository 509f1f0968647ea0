"""Writes tests/golden/container_small.bin with the REFERENCE's own Python tools.

Run where the reference checkout is present:

    python tests/golden/make_container_fixture.py /path/to/fish-audio-cpp

It imports the reference's ``tools/quant_utils.py`` (numpy only), quantises a few seeded fp32 matrices with its
``quantize_groupwise``, lays the entries out the way ``tools/step2_export_w8a8.py:207-271`` does (headers, then each
tensor at the next multiple of 256), writes the headers with its ``write_headers_only`` and appends the data. The
result pins this repo's reader and writer (``fish-audio-cpp_b200/container.py``) to the reference's file format.
The tensors are small on purpose (the file is about 60 KB); names follow the engine's loader.
"""
import importlib.util
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def tensors(qu):
    """name -> (dtype_val, array), in file order. fp32 sources are seeded; int8 and scales come from the reference."""
    rng = np.random.default_rng(20240607)
    p = "text_model.model.layers.0."
    out = {}

    def quantized(name, n, k, group, smooth=None):
        w = rng.standard_normal((n, k)).astype(np.float32) * 0.05
        q, s = qu.quantize_groupwise(w, group)
        out[name] = (3, q)
        out[name + "_scale"] = (1, s)
        if smooth is not None:
            out[name + "_smooth_inv"] = (1, smooth)

    out[p + "attention_norm.weight"] = (1, (1.0 + 0.1 * rng.standard_normal(512)).astype(np.float16))
    smooth = rng.uniform(0.5, 2.0, 512).astype(np.float16)
    quantized(p + "attention.wqkv.weight", 48, 512, 256)
    quantized(p + "attention.wo.weight", 32, 256, 64)
    quantized(p + "feed_forward.w1.weight", 32, 512, 256, smooth)
    quantized(p + "feed_forward.w3.weight", 32, 512, 256, smooth)
    quantized(p + "feed_forward.w2.weight", 16, 300, 512)  # one group: the scale is [N]
    out["audio_decoder.norm.weight"] = (0, rng.standard_normal(7).astype(np.float32))
    return out


def main(reference_root: str) -> None:
    spec = importlib.util.spec_from_file_location("ref_quant_utils", Path(reference_root) / "tools" / "quant_utils.py")
    qu = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(qu)
    ts = tensors(qu)
    entries = []
    for name, (code, arr) in ts.items():
        entries.append({"name": name, "dtype_val": code, "shape": list(arr.shape), "data_size": arr.nbytes})
    cur = qu.align256(12 + qu.HEADER_SIZE * len(entries))
    for e in entries:
        e["data_offset"] = cur
        cur = qu.align256(cur + e["data_size"])
    path = HERE / "container_small.bin"
    data_start = qu.write_headers_only(entries, str(path))
    assert data_start == entries[0]["data_offset"]
    with open(path, "r+b") as f:
        for e, (name, (code, arr)) in zip(entries, ts.items()):
            f.seek(e["data_offset"])
            f.write(np.ascontiguousarray(arr).tobytes())
        f.truncate(max(f.tell(), entries[-1]["data_offset"] + entries[-1]["data_size"]))
    np.savez_compressed(HERE / "container_small_expected.npz", **{k: v[1] for k, v in ts.items()})
    print(path, path.stat().st_size, "bytes,", len(entries), "tensors")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
