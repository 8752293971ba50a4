"""Writes tests/golden/plain_anchors.json: literal input/output pairs of the parts.

The reference is a Rust workspace and no Rust toolchain exists where this was made, so its
model code could not be run; these anchors rest on the formulas alone.  Each case restates
a literal test of the reference (crates/sglang-kernel/tests/cpu_kernels.rs:10-80 for the norm,
the projection and the rotations; crates/sglang-srt/tests/cuda_inference.rs:326-416 with :86
for the one-hot model whose greedy continuation of [1] is [2, 1]) with the expected values
worked out by hand from the formula, in plain Python floats, not by the functions under
test.  Run: python tests/golden/make_golden.py
"""
import json
import math
import os


def main():
    cos, sin = math.cos(1.0), math.sin(1.0)
    s0 = math.sqrt((1.0 + 4.0) / 2 + 1e-6)
    s1 = math.sqrt((9.0 + 16.0) / 2 + 1e-6)
    g = [0.5, -1.0, 2.0]
    u = [2.0, 3.0, -1.5]
    anchors = {
        "rms_norm": {"x": [[1.0, 2.0], [3.0, 4.0]], "w": [1.0, 0.5], "eps": 1e-6,
                     "y": [[1.0 / s0, 2.0 / s0 * 0.5], [3.0 / s1, 4.0 / s1 * 0.5]]},
        "linear": {"x": [[1.0, 2.0], [3.0, 4.0]], "w": [[1.0, 0.0], [0.0, 1.0], [1.0, 1.0]],
                   "b": [0.5, -0.5, 1.0], "y": [[1.5, 1.5, 4.0], [3.5, 3.5, 8.0]]},
        "rope_neox": {"x": [1.0, 2.0, 3.0, 4.0], "position": 1, "theta": 1.0,
                      "y": [1 * cos - 3 * sin, 2 * cos - 4 * sin, 3 * cos + 1 * sin, 4 * cos + 2 * sin]},
        "silu_mul": {"g": g, "u": u, "y": [gi / (1 + math.exp(-gi)) * ui for gi, ui in zip(g, u)]},
        "one_hot_model": {"prompt": [1], "greedy": [2, 1]},
    }
    # attention: one query head on two kv positions, d = 2, scale 1/sqrt(2)
    q, k0, k1, v0, v1 = [1.0, 0.0], [1.0, 0.0], [0.0, 1.0], [1.0, 2.0], [3.0, 4.0]
    scale = 1 / math.sqrt(2)
    e0, e1 = math.exp(scale * 1.0 - scale), math.exp(0.0 - scale)
    anchors["attention"] = {"q": q, "k": [k0, k1], "v": [v0, v1], "scale": scale,
                            "y_last": [(e0 * v0[i] + e1 * v1[i]) / (e0 + e1) for i in range(2)], "y_first": v0}
    # literal vectors of the reference's own tests, copied as data:
    # grouped-query attention of one token, four query heads on two kv heads, scale 1
    # (crates/sglang-kernel/tests/cpu_kernels.rs:174-190)
    anchors["gqa_one_token"] = {"q": [1.0, 0.0, 0.0, 1.0, 1.0, 0.0, 0.0, 1.0], "k": [1.0, 0.0, 0.0, 1.0],
                                "v": [2.0, 3.0, 5.0, 7.0], "query_heads": 4, "kv_heads": 2, "head_dim": 2,
                                "scale": 1.0, "y": [2.0, 3.0, 2.0, 3.0, 5.0, 7.0, 5.0, 7.0]}
    # the k largest probabilities of a row, renormalised (cpu_kernels.rs:200-238)
    anchors["top_k_renorm"] = {"probs": [[0.1, 0.2, 0.7, 0.4], [0.3, 0.2, 0.1, 0.0]],
                               "fixed_k": 2, "fixed_y": [[0.0, 0.0, 7.0 / 11.0, 4.0 / 11.0], [3.0 / 5.0, 2.0 / 5.0, 0.0, 0.0]],
                               "per_row_k": [1, 3],
                               "per_row_y": [[0.0, 0.0, 1.0, 0.0], [3.0 / 6.0, 2.0 / 6.0, 1.0 / 6.0, 0.0]]}
    # rotation of the first four of six values only (cpu_kernels.rs:63-80)
    anchors["rope_partial"] = {"x": [1.0, 2.0, 3.0, 4.0, 5.0, 6.0], "rotary_dim": 4, "position": 1, "theta": 1.0,
                               "y": [1 * cos - 3 * sin, 2 * cos - 4 * sin, 3 * cos + 1 * sin, 4 * cos + 2 * sin, 5.0, 6.0]}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "plain_anchors.json")
    with open(path, "w") as handle:
        json.dump(anchors, handle, indent=1)
    print("wrote", path)


if __name__ == "__main__":
    main()
