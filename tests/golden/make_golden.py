"""Regenerates the fixtures in this directory.

Two kinds of fixture live here:

* the reference's own golden vectors for the quantized-linear path, taken from
  a TensorPencil checkout (``--reference PATH``):
  the ComfyUI int4 ConvRot dequant fixture (``testdata/int4_convrot_*``, used by
  the test in ``src/ops/convrot.zig:148-192``) and the ggml Q8_0 dequant block
  with its expected f32 bit patterns (``src/core/quants_fixtures.zig:6-15``) and the
  q4_k / q5_k / q6_k super-blocks of the same file;
* small seeded input/output vectors produced by the CPU oracle, so a change in
  the oracle's arithmetic shows up as a diff against a committed file.

Run from the repository root:  python tests/golden/make_golden.py
"""
import argparse
import json
import os
import re
import shutil
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)


def copy_reference_fixtures(ref: str) -> None:
    for name in ("int4_convrot_weight.u8", "int4_convrot_scale.f32", "int4_convrot_expected.f32"):
        shutil.copyfile(os.path.join(ref, "testdata", name), os.path.join(HERE, name))
    src = open(os.path.join(ref, "src/core/quants_fixtures.zig")).read()

    def table(name):
        body = re.search(r"pub const %s = \[_\]u\d+\{(.*?)\};" % name, src, re.S).group(1)
        return [int(t, 16) for t in re.findall(r"0x[0-9a-fA-F]+", body)]

    with open(os.path.join(HERE, "q8_0_block.json"), "w") as f:
        json.dump({"source": "src/core/quants_fixtures.zig:6-15",
                   "block_bytes": table("q8_0_block"),
                   "expected_f32_bits": table("q8_0_expected_bits")}, f, indent=1)
    # k-quant super-blocks (256 elements) with ggml's expected dequantisation
    with open(os.path.join(HERE, "kquant_blocks.json"), "w") as f:
        json.dump({"source": "src/core/quants_fixtures.zig:18-160",
                   **{fmt: {"block_bytes": table(fmt + "_block"), "expected_f32_bits": table(fmt + "_expected_bits")}
                      for fmt in ("q4_k", "q5_k", "q6_k")}}, f)


def oracle_vectors() -> None:
    from oracle import oracle
    from tensorpencil_b200 import synth

    out = {}
    # ConvRot prep + int GEMM + dequant, both widths, small shapes with an outlier channel.
    for bits in (8, 4):
        c = synth.convrot_linear(m=5, n=24, k=512, bits=bits, seed=4200 + bits)
        q, s, acc, y = oracle.convrot_linear_sim(c["x"], c["w_i8"], c["w_scale"], bits)
        out[f"i{bits}_x"] = c["x"]
        out[f"i{bits}_w"] = c["w_i8"]
        out[f"i{bits}_ws"] = c["w_scale"]
        out[f"i{bits}_q"] = q
        out[f"i{bits}_as"] = s
        out[f"i{bits}_acc"] = acc
        out[f"i{bits}_y"] = y
        out[f"i{bits}_cpu_backend"] = oracle.linear_cpu_backend(
            c["x"], c["w_packed"] if bits == 4 else c["w_i8"], bits, c["w_scale"], 24, 512)
    # Q8_0 GEMV, M = 3 activation rows.
    g = synth.q8_0_gemv(m=3, n=16, k=512, seed=4300)
    out["q8_w"] = g["w"]
    out["q8_x"] = g["x"]
    out["q8_y_f64"] = oracle.q8_0_gemv_f64(g["w"], 16, 512, g["x"])
    out["q8_y_q8"] = oracle.q8_0_gemv_q8(g["w"], 16, 512, g["x"])
    d, qs = oracle.q8_1_quantize(g["x"])
    out["q8_act_d"] = d
    out["q8_act_qs"] = qs
    np.savez_compressed(os.path.join(HERE, "oracle_vectors.npz"), **out)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a TensorPencil checkout")
    a = ap.parse_args()
    if os.path.isdir(a.reference):
        copy_reference_fixtures(a.reference)
    else:
        print("reference checkout not found; keeping the committed reference fixtures")
    oracle_vectors()
