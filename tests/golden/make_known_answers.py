"""Writes reference_known_answers.json: the exact expectations that the reference's own tests
hold for the GEMM path, transcribed as data (inputs, operation, expected output, source).

Sources (paths inside the reference project):
  gradtuity/tests/test_tensor.py:1729-1875   TestMatmul
  gradtuity/tests/test_nn.py:1165-1279       TestFusedLinear
  gradtuity/tests/test_nn.py:1291-1450       TestLinearRelu
All values are small integers or short decimals, exactly representable in tf32 or within
pytest.approx's default 1e-6 relative tolerance of it, so they hold for every precision mode.

Run:  python tests/golden/make_known_answers.py
"""
import json
import os

CASES = [
    # ---- TestMatmul -----------------------------------------------------------------
    {"name": "matmul_forward_small", "src": "gradtuity/tests/test_tensor.py:1729-1745", "op": "matmul",
     "a": [[1, 2, 3], [4, 5, 6]], "b": [[1, 2], [3, 4], [5, 6]], "y": [[22, 28], [49, 64]]},
    {"name": "matmul_forward_identity", "src": "gradtuity/tests/test_tensor.py:1747-1756", "op": "matmul",
     "a": [[1, 2], [3, 4]], "b": [[1, 0], [0, 1]], "y": [[1, 2], [3, 4]]},
    {"name": "matmul_forward_batch_vector", "src": "gradtuity/tests/test_tensor.py:1758-1789", "op": "matmul",
     "a": [[1, 0, 0], [0, 1, 0], [0, 0, 1], [1, 1, 1]], "b": [[1, 2], [3, 4], [5, 6]],
     "y": [[1, 2], [3, 4], [5, 6], [9, 12]]},
    {"name": "matmul_backward_a_only", "src": "gradtuity/tests/test_tensor.py:1807-1822", "op": "matmul_sum_backward",
     "a": [[1, 2], [3, 4]], "b": [[1, 0], [0, 1]], "a_grad": True, "b_grad": False,
     "da": [[1, 1], [1, 1]], "db": None},
    {"name": "matmul_backward_b_only", "src": "gradtuity/tests/test_tensor.py:1824-1839", "op": "matmul_sum_backward",
     "a": [[1, 0], [0, 1]], "b": [[1, 2], [3, 4]], "a_grad": False, "b_grad": True,
     "da": None, "db": [[1, 1], [1, 1]]},
    {"name": "matmul_backward_both", "src": "gradtuity/tests/test_tensor.py:1841-1865", "op": "matmul_sum_backward",
     "a": [[1, 2, 3], [4, 5, 6]], "b": [[1, 2], [3, 4], [5, 6]], "a_grad": True, "b_grad": True,
     "da": [[3, 7, 11], [3, 7, 11]], "db": [[5, 5], [7, 7], [9, 9]]},
    # ---- TestFusedLinear --------------------------------------------------------------
    {"name": "linear_forward", "src": "gradtuity/tests/test_nn.py:1165-1179", "op": "linear",
     "x": [[1, 0, 0], [0, 1, 0]], "w": [[1, 2], [3, 4], [5, 6]], "bias": [0.1, 0.2], "y": [[1.1, 2.2], [3.1, 4.2]]},
    {"name": "linear_backward_db", "src": "gradtuity/tests/test_nn.py:1199-1220", "op": "linear_sum_backward",
     "x": [[1, 2]], "w": [[0.5, 1.0], [1.5, 2.0]], "bias": [0.1, 0.2], "dbias": [1, 1]},
    {"name": "linear_backward_x_only", "src": "gradtuity/tests/test_nn.py:1222-1238", "op": "linear_sum_backward",
     "x": [[1, 2], [3, 4]], "w": [[1, 0], [0, 1]], "bias": [0, 0], "dx": [[1, 1], [1, 1]]},
    # ---- TestLinearRelu ---------------------------------------------------------------
    {"name": "linear_relu_forward", "src": "gradtuity/tests/test_nn.py:1291-1306", "op": "linear_relu",
     "x": [[1, 0], [0, 1]], "w": [[1, -1], [2, -2]], "bias": [0.5, 0.5], "y": [[1.5, 0], [2.5, 0]]},
    {"name": "linear_relu_all_positive", "src": "gradtuity/tests/test_nn.py:1326-1335", "op": "linear_relu",
     "x": [[1, 1]], "w": [[1, 1], [1, 1]], "bias": [1, 1], "y": [[3, 3]]},
    {"name": "linear_relu_all_negative", "src": "gradtuity/tests/test_nn.py:1337-1346", "op": "linear_relu",
     "x": [[1, 1]], "w": [[-1, -1], [-1, -1]], "bias": [-1, -1], "y": [[0, 0]]},
    {"name": "linear_relu_backward_x_only", "src": "gradtuity/tests/test_nn.py:1397-1418", "op": "linear_relu_sum_backward",
     "x": [[1, 2]], "w": [[1, 0], [0, 1]], "bias": [0, -10], "dx": [[1, 0]]},
    {"name": "linear_relu_blocks_gradient", "src": "gradtuity/tests/test_nn.py:1420-1441", "op": "linear_relu_sum_backward",
     "x": [[1]], "w": [[-1, 1]], "bias": [0, 0], "dw": [[0, 1]], "dbias": [0, 1]},
]

if __name__ == "__main__":
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_known_answers.json")
    with open(out, "w") as f:
        json.dump(CASES, f, indent=1)
    print("wrote", out, len(CASES), "cases")
