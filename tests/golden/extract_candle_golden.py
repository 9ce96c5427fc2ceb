"""Extracts the golden vectors that candle's own tests hold for the norm + embedding path.

Run in a checkout that has the reference mounted:

    python tests/golden/extract_candle_golden.py <candle checkout> tests/golden/candle_kats.json

It READS the reference's test sources as text (no Rust toolchain is needed), pulls the numeric array
literals out of the named test functions and writes them, with the file:line they came from, to a
JSON fixture.  The fixture is committed; the GPU box never sees the reference tree.
"""
from __future__ import annotations

import json
import re
import sys


def function_body(text: str, name: str) -> tuple[str, int]:
    """Body of ``fn <name>(`` found by brace matching, with the 1-based line of the ``fn``."""
    m = re.search(r"\bfn\s+" + re.escape(name) + r"\s*\(", text)
    if m is None:
        raise KeyError(name)
    start = text.index("{", m.end())
    depth, i = 0, start
    while True:
        c = text[i]
        if c == "{":
            depth += 1
        elif c == "}":
            depth -= 1
            if depth == 0:
                break
        i += 1
    return text[start : i + 1], text.count("\n", 0, m.start()) + 1


def array_literals(body: str) -> list:
    """Every bracket-balanced ``[...]`` literal of the body that parses as nested numbers."""
    body = re.sub(r"//[^\n]*", "", body)
    out, i = [], 0
    while i < len(body):
        if body[i] == "[":
            depth, j = 0, i
            while True:
                if body[j] == "[":
                    depth += 1
                elif body[j] == "]":
                    depth -= 1
                    if depth == 0:
                        break
                j += 1
            lit = body[i : j + 1]
            lit = re.sub(r"(?<=[0-9.])(f32|f64|u32|u8|i64)\b", "", lit)  # 3f32 -> 3, 0.5f32 -> 0.5
            lit = re.sub(r"(\d)\.(?=[\s,\]])", r"\1.0", lit)  # 1. -> 1.0
            lit = re.sub(r",\s*\]", "]", lit)  # trailing commas
            try:
                val = json.loads(lit)
                out.append(val)
                i = j + 1
                continue
            except json.JSONDecodeError:
                pass
        i += 1
    return out


def main(ref: str, dst: str) -> None:
    def read(rel):
        with open(f"{ref}/{rel}") as f:
            return f.read()

    kats = {}

    ops = read("candle-nn/tests/ops.rs")
    body, line = function_body(ops, "rms_norm")
    lits = array_literals(body)
    kats["rms_norm"] = {
        "source": f"candle-nn/tests/ops.rs:{line}", "x": lits[0], "alpha": lits[1], "eps": 1e-5,
        "expected_round4": lits[2], "expected_slow_round4": lits[3],
    }
    body, line = function_body(ops, "layer_norm")
    lits = array_literals(body)
    kats["layer_norm"] = {
        "source": f"candle-nn/tests/ops.rs:{line}", "x": lits[0], "alpha": lits[1], "beta": lits[2], "eps": 1e-5,
        "expected_round4": lits[3], "expected_slow_round4": lits[4],
    }
    for name in ("rms_norml", "layer_norml"):
        body, line = function_body(ops, name)
        dims = re.search(r"=\s*\((\d+),\s*(\d+),\s*(\d+)\)", body)
        kats[name] = {
            "source": f"candle-nn/tests/ops.rs:{line}", "shape": [int(g) for g in dims.groups()],
            "distribution": "uniform[0,1)", "eps": 1e-5, "max_abs_fused_vs_slow": 1e-5,
        }

    # softmax: the test takes log(data) and applies softmax over each dim; the last-dim values are the
    # ones softmax_last_dim is checked against (third and fourth expected blocks, identical)
    body, line = function_body(ops, "softmax")
    lits = array_literals(body)
    assert lits[3] == lits[4]
    kats["softmax"] = {
        "source": f"candle-nn/tests/ops.rs:{line}", "data": lits[0], "input": "log(data)",
        "expected_dim0_round4": lits[1], "expected_dim1_round4": lits[2], "expected_last_dim_round4": lits[4],
    }
    body, line = function_body(ops, "softmax_numerical_stability")
    lits = array_literals(body)
    kats["softmax_numerical_stability"] = {"source": f"candle-nn/tests/ops.rs:{line}", "x": lits[0], "expected": lits[1]}
    for name in ("ropei", "rope", "rope_thd"):
        body, line = function_body(ops, name)
        dims = re.search(r"=\s*\((\d+),\s*(\d+),\s*(\d+),\s*(\d+)\)", body)
        kats[name] = {
            "source": f"candle-nn/tests/ops.rs:{line}", "b_size_num_head_seq_len_head_dim": [int(g) for g in dims.groups()],
            "distribution": "uniform[0,1) for src, cos and sin", "fused_vs_slow_sum_abs_diff": 0.0,
        }

    ln = read("candle-nn/tests/layer_norm.rs")
    body, line = function_body(ln, "layer_norm")
    lits = array_literals(body)
    # order in the source: w, b, (cat lists are not numeric), two, [0.5], inp2, expected2, inp3, expected3, mean, std
    nums = [l for l in lits if l and not isinstance(l[0], str)]
    kats["layer_norm_module"] = {
        "source": f"candle-nn/tests/layer_norm.rs:{line}", "w": nums[0], "b": nums[1], "eps": 1e-8,
        "cases": [
            {"x": nums[2], "expected": nums[3], "exact": True},
            {"x": nums[4], "expected": nums[5], "exact": True},
            {"x": nums[6], "expected_round4": nums[7], "mean_round4": nums[8], "std_round4": nums[9]},
        ],
    }

    doc = read("candle-nn/src/layer_norm.rs")
    head = doc[: doc.index("\nuse candle::")]
    head = "\n".join(l[3:] if l.startswith("//!") else l for l in head.splitlines())
    lits = array_literals(head)
    kats["layer_norm_doctest"] = {
        "source": "candle-nn/src/layer_norm.rs:7-28", "w": lits[0], "b": lits[1], "eps": 1e-5,
        "x": lits[2], "expected_round4": lits[3],
    }

    tt = read("candle-core/tests/tensor_tests.rs")
    body, line = function_body(tt, "embeddings")
    lits = array_literals(body)
    kats["embeddings"] = {
        "source": f"candle-core/tests/tensor_tests.rs:{line}", "ids": lits[0], "table": lits[1], "expected": lits[2],
    }
    body, line = function_body(tt, "index_select")
    lits = array_literals(body)
    kats["index_select"] = {
        "source": f"candle-core/tests/tensor_tests.rs:{line}",
        "ids": lits[0], "table_arange": [4, 3], "table": lits[1],
        "expected_dim1": lits[2], "expected_dim0": lits[3],
        "ids_repeated": lits[4], "expected_repeated_dim0": lits[5],
        "ids2": lits[6], "table2": lits[7], "expected2_dim1": lits[8],
        "id_dtypes": ["u8", "u32", "i64"],
    }

    qt = read("candle-core/tests/quantized_tests.rs")
    body, line = function_body(qt, "quantize_q4_0")
    lits = array_literals(body)
    vec = max(lits, key=len)
    assert len(vec) == 128
    kats["quantize_q4_0"] = {
        "source": f"candle-core/tests/quantized_tests.rs:{line}", "src": "0..128 as f32",
        "dequantized": [repr(float(v)) for v in vec],  # strings keep the sign of -0.0
    }

    # the other 32-element block formats: same test shape, values compared after rounding to 3 decimals
    for name in ("quantize_q4_1", "quantize_q5_0", "quantize_q5_1"):
        body, line = function_body(qt, name)
        vec = max(array_literals(body), key=len)
        assert len(vec) == 128
        kats[name] = {
            "source": f"candle-core/tests/quantized_tests.rs:{line}", "src": "0..128 as f32",
            "dequantized_rounded_3": [repr(float(v)) for v in vec],
            "rounding": "(1000 * x).round() / 1000 in f32, round half away from zero (round_vector)",
        }

    # K-quant super-blocks: a 1024-element ramp of bound 0.5 quantised and decoded again; candle checks
    # six decoded values (rounded to 3 decimals), a max-abs error over the vector, the same for a ramp
    # of bound 128, and an RMSE bound on the cosine vector of the ggml unit tests
    consts = dict(re.findall(r"const (GGML_MAX_QUANTIZATION_TOTAL_ERROR\w*): f32 = ([0-9.]+);", qt))
    test_size = re.search(r"const GGML_TEST_SIZE: usize = ([0-9* ]+);", qt).group(1)
    for name in ("quantize_q2k", "quantize_q3k", "quantize_q4k", "quantize_q5k", "quantize_q6k", "quantize_q8k"):
        body, line = function_body(qt, name)
        lits = [l for l in array_literals(body) if len(l) == 6]
        tols = [float(t) for t in re.findall(r"compare_with_error\([^;]*?,\s*([0-9.]+)\s*\)", body)]
        vecs = re.findall(r"get_test_vector2\(([0-9.]+),\s*(\d+),", body)
        rmse = re.search(r"ggml_quantization_error_test\(dtype, device, (\w+)\)", body).group(1)
        kats[name] = {
            "source": f"candle-core/tests/quantized_tests.rs:{line}",
            "src": "get_test_vector2(bound, size): ((v - size/2) * bound) / (size/2) in f32, v in 0..size",
            "bound": float(vecs[0][0]), "size": int(vecs[0][1]), "points": [0, 128, 256, 512, 800, 1023],
            "src_points": [repr(float(v)) for v in lits[0]],
            "dequantized_points_rounded_3": [repr(float(v)) for v in lits[1]],
            "max_abs_error": tols[0], "big_bound": float(vecs[1][0]), "big_max_abs_error": tols[1],
            "ggml_vector": f"0.1 + 2 cos(i) for i in 0..{eval(test_size)}", "ggml_size": eval(test_size),
            "ggml_max_rmse": float(consts[rmse]),
            "rmse": "sqrt(sum((a - b)^2)) / len",
        }

    with open(dst, "w") as f:
        json.dump(kats, f, indent=1)
    print(f"wrote {dst}: {sorted(kats)}")


if __name__ == "__main__":
    main(sys.argv[1], sys.argv[2])
