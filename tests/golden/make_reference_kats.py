"""Writes reference_kats.json: the known-answer vectors of the reference's own tests for the GGML
quantized dense / gather path, transcribed as bytes.

Sources (gomlx/gomlx):
  ml/nn/quantized_dense_test.go:272-334   TestQuantizedDense_GGML_Q8_0  (basic, with_bias, batch)
  ml/nn/quantized_dense_test.go:340-401   TestQuantizedDense_GGML_Q4_0  (basic, with_silu)
  ml/nn/quantized_gather_test.go:17-74    TestQuantizedGather_GGML_Q8_0 (basic, single)
  ml/nn/quantized_gather_test.go:78-121   TestQuantizedGather_GGML_Q4_0 (basic)

The reference is Go and cannot be executed here, so these are the vectors written in its test
source, not outputs of a run.  Run: python tests/golden/make_reference_kats.py
"""
import json
import os

Q4_0, Q8_0 = 2, 8


def q8_row(scale_hi_byte, ones):
    row = [0] * 34
    row[0], row[1] = 0x00, scale_hi_byte
    for i in ones:
        row[2 + i] = 1
    return row


def q4_row(scale_hi_byte, nine_at):
    row = [0x88] * 18
    row[0], row[1] = 0x00, scale_hi_byte
    row[2 + nine_at] = 0x89
    return row


def onehot(n, pairs):
    v = [0.0] * n
    for i, x in pairs:
        v[i] = x
    return v


x11 = onehot(32, [(0, 1.0), (1, 1.0)])
w8 = [q8_row(0x40, [0]), q8_row(0x42, [1])]
w4 = [q4_row(0x40, 0), q4_row(0x42, 1)]
t8 = [q8_row(0x40, [0]), q8_row(0x42, [1]), q8_row(0x3C, [0, 1])]

kats = {
    "dense": [
        {"name": "Q8_0/basic", "src": "ml/nn/quantized_dense_test.go:296-306", "type": Q8_0, "w": w8, "x": [x11],
         "bias": None, "act": "none", "want": [[2.0, 3.0]], "delta": 1e-4},
        {"name": "Q8_0/with_bias", "src": "ml/nn/quantized_dense_test.go:309-319", "type": Q8_0, "w": w8, "x": [x11],
         "bias": [0.5, -0.5], "act": "none", "want": [[2.5, 2.5]], "delta": 1e-4},
        {"name": "Q8_0/batch", "src": "ml/nn/quantized_dense_test.go:322-333", "type": Q8_0, "w": w8,
         "x": [x11, onehot(32, [(0, 0.5)])], "bias": None, "act": "none", "want": [[2.0, 3.0], [1.0, 0.0]],
         "delta": 1e-4},
        {"name": "Q4_0/basic", "src": "ml/nn/quantized_dense_test.go:373-383", "type": Q4_0, "w": w4, "x": [x11],
         "bias": None, "act": "none", "want": [[2.0, 3.0]], "delta": 1e-4},
        {"name": "Q4_0/with_silu", "src": "ml/nn/quantized_dense_test.go:386-400", "type": Q4_0, "w": w4, "x": [x11],
         "bias": None, "act": "silu", "want": [[1.7616, 2.8577]], "delta": 1e-3},
    ],
    "gather": [
        {"name": "Q8_0/basic", "src": "ml/nn/quantized_gather_test.go:49-58", "type": Q8_0, "table": t8,
         "indices": [[2], [0]], "want": [onehot(32, [(0, 1.0), (1, 1.0)]), onehot(32, [(0, 2.0)])], "delta": 1e-4},
        {"name": "Q8_0/single", "src": "ml/nn/quantized_gather_test.go:64-73", "type": Q8_0, "table": t8,
         "indices": [[1]], "want": [onehot(32, [(1, 3.0)])], "delta": 1e-4},
        {"name": "Q4_0/basic", "src": "ml/nn/quantized_gather_test.go:110-119", "type": Q4_0, "table": w4,
         "indices": [[1], [0]], "want": [onehot(32, [(1, 3.0)]), onehot(32, [(0, 2.0)])], "delta": 1e-4},
    ],
}

if __name__ == "__main__":
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_kats.json")
    with open(out, "w") as f:
        json.dump(kats, f)
    print(out)
