"""Transcribe the `// EXPECT-OUT:` lines of the reference's hot-path fixtures into expect_out.json.

Run once, where the reference tree is mounted:

    python tests/golden/extract_expect_out.py /path/to/reference

The reference states that these values are "scalar semantics computed independently, never recorded
output" (tests/README.md of the reference), which is what makes them golden vectors for the oracle.
Only the numbers are taken; the tests rebuild each fixture's inputs from its documented construction.
"""
import json
import os
import sys

FIXTURES = [
    "builtin_activations", "builtin_norms", "builtin_matmul", "decode_gemv_half", "decode_gemv_quant",
    "int4_dequant", "decode_kv_attention", "decode_kv_batch", "decode_kv_batch_gqa", "sdpa", "rope",
    "norm_blocked_every_lane", "decode_tiny_lm", "embedding", "rowargmax", "cov4_par_decode",
    "linear_bf16", "f8_code_round_trip", "gemv_f32", "softmax", "rmsnorm", "layernorm", "gelu",
]


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: extract_expect_out.py <path of the reference checkout>")
    ref = sys.argv[1]
    out = {}
    for name in FIXTURES:
        path = os.path.join(ref, "tests", "run", name + ".wk")
        lines = []
        with open(path) as fh:
            for ln in fh:
                if ln.startswith("// EXPECT-OUT:"):
                    lines.append(ln[len("// EXPECT-OUT:"):].strip())
        out[name] = lines
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "expect_out.json")
    with open(dst, "w") as fh:
        json.dump(out, fh, indent=0)
    print("wrote", dst, {k: len(v) for k, v in out.items()})


if __name__ == "__main__":
    main()
