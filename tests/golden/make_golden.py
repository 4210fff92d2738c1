"""Generate the golden fixtures of tests/golden/ from the reference itself.

Run in a container where the reference checkout is available (CPU only is fine):

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's Python package on CPU (no GPU needed for these parts):

* cast_kat.npz   - every code of every sub-byte float / int type decoded by the
                   reference's known-answer functions cast_fx_to_f32_ref and
                   cast_ix_to_i32_ref, and cast_f32_to_fx_ref on the reference's
                   2001 rounding probes (tests/kernels/test_cast.py:44-82, :93-145,
                   :200-225 of the reference).
* tile_layout.npz- for b = 1..8, the placement of every element of a 16x16 weight
                   tile in the reference's re-laid-out weight format, obtained from
                   the reference's layout algebra (tilus.ir.layout) exactly as
                   QuantizedMatmulCommon builds it (examples/quantization/matmul_a16wx.py:29-61).
* dtype_meta.json- nbits / min / max of the reference's dtype objects.

The fixtures are small and committed; tests only read the fixtures.
"""
import importlib.util
import json
import math
import os
import sys
import tempfile

import numpy as np


def _import_reference(ref_root: str):
    stub = tempfile.mkdtemp(prefix="tilus_stub_")
    os.makedirs(os.path.join(stub, "tilus-0.2.0.dist-info"))
    with open(os.path.join(stub, "tilus-0.2.0.dist-info", "METADATA"), "w") as f:
        f.write("Metadata-Version: 2.1\nName: tilus\nVersion: 0.2.0\n")
    sys.dont_write_bytecode = True
    sys.path.insert(0, stub)
    sys.path.insert(0, os.path.join(ref_root, "python"))
    import tilus  # noqa: F401

    spec = importlib.util.spec_from_file_location(
        "ref_test_cast", os.path.join(ref_root, "tests", "kernels", "test_cast.py")
    )
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return tilus, mod


FLOAT_NAMES = [
    "float7_e5m1", "float7_e4m2", "float7_e3m3", "float7_e2m4",
    "float6_e4m1", "float6_e3m2", "float6_e2m3",
    "float5_e3m1", "float5_e2m2", "float5_e1m3",
    "float4_e2m1", "float4_e1m2", "float3_e1m1",
]
INT_NAMES = [f"int{n}b" for n in range(1, 8)] + [f"uint{n}b" for n in range(1, 8)]


def main():
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TILUS_REFERENCE_ROOT")
    if not ref_root:
        sys.exit("usage: make_golden.py <root of the reference checkout>  (or set TILUS_REFERENCE_ROOT)")
    out_dir = os.path.dirname(os.path.abspath(__file__))
    tilus, kat = _import_reference(ref_root)
    import tilus.hidet.ir.dtypes as D

    arrays = {}
    meta = {}
    for name in FLOAT_NAMES:
        dt = getattr(D.floats_subbyte, name)
        nb = dt.nbits
        arrays[f"decode/{name}"] = np.array(
            [kat.cast_fx_to_f32_ref(c, dt) for c in range(1 << nb)], dtype=np.float64
        )
        probes = [i / 1000 for i in range(1000)] + [i / 1000 * float(dt.max_value) for i in range(1001)]
        probes = np.array(probes, dtype=np.float32)
        arrays[f"probes/{name}"] = probes
        arrays[f"encode/{name}"] = np.array(
            [kat.cast_f32_to_fx_ref(float(p), dt) for p in probes], dtype=np.int64
        )
        meta[name] = dict(nbits=nb, e=dt.exponent_nbits, m=dt.mantissa_nbits,
                          min=float(dt.min_value), max=float(dt.max_value))
    for name in INT_NAMES:
        dt = getattr(D.integer_subbyte, name)
        nb = dt.nbits
        arrays[f"decode/{name}"] = np.array(
            [kat.cast_ix_to_i32_ref(c, dt) for c in range(1 << nb)], dtype=np.float64
        )
        meta[name] = dict(nbits=nb, signed=bool(dt.signedness()),
                          min=int(dt.min_value), max=int(dt.max_value))
    np.savez_compressed(os.path.join(out_dir, "cast_kat.npz"), **arrays)
    with open(os.path.join(out_dir, "dtype_meta.json"), "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)

    # ---- weight-tile placement from the reference's layout algebra ------------
    from tilus.ir.instructions.cuda.mma_dot import AtomicMmaConfig
    from tilus.ir.layout.ops import local

    lb = AtomicMmaConfig.m16n8k16_f16_f32().lb
    tile_layout = local(16 // 16, 16 // 8) * lb
    lane = np.zeros((16, 16), dtype=np.int64)
    slot = np.zeros((16, 16), dtype=np.int64)
    for k in range(16):
        for n in range(16):
            lane[k, n] = int(tile_layout.get_spatial([k, n])[0])
            slot[k, n] = int(tile_layout.get_local([k, n]))
    tl = {"lane": lane, "slot": slot}
    for b in range(1, 9):
        bytes_per_thread = tile_layout.local_size * b // 8
        inner = math.gcd(bytes_per_thread, 16)
        outer = bytes_per_thread // inner
        flat = local(outer).spatial(32).local(inner)
        size = int(flat.shape[0])
        assert size == 32 * b
        fl_lane = np.array([int(flat.get_spatial([p])[0]) for p in range(size)], dtype=np.int64)
        fl_local = np.array([int(flat.get_local([p])) for p in range(size)], dtype=np.int64)
        tl[f"flat_lane/{b}"] = fl_lane
        tl[f"flat_local/{b}"] = fl_local
    np.savez_compressed(os.path.join(out_dir, "tile_layout.npz"), **tl)
    print("wrote", sorted(os.listdir(out_dir)))


if __name__ == "__main__":
    main()
