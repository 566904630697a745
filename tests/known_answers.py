"""Known-answer vectors of the reference's own unit tests for the training hot path, restated as data.

Each case cites the reference test it comes from (paths relative to the reference repository). They are
used twice: ``test_oracle_pins.py`` pins the numpy oracle to them on CPU, and the ``-m gpu`` tests run the
same cases through the C ABI of ``libcgpt_b200.so``.
"""
import math

import numpy as np

E = math.exp

# tests/cut_cross_entropy_test.cu:19-31 (F32; tolerance 2e-5, classifier gradient 2e-3)
CCE = dict(
    input=np.array([[1, 2], [3, 4]], np.float32),
    classifier=np.array([[1, 0], [0, 1], [1, 1]], np.float32),
    targets=np.array([2, 0], np.uint32),
    loss=(math.log(E(1) + E(2) + E(3)) - 3.0 + math.log(E(3) + E(4) + E(7)) - 3.0) / 2,
    grad_input=np.array([[-0.1223642, -0.0450153], [-0.0234640, 0.4915309]], np.float32),
    grad_classifier=np.array([[-1.429500, -1.876000], [0.193000, 0.339000], [1.736500, 2.537000]], np.float32),
)

# tests/cross_entropy_test.cu:33-56 (F32; tolerance 1e-5)
CE = dict(
    logits=np.array([[1, 2, 3], [1, 1, 1]], np.float32),
    targets=np.array([2, 0], np.uint32),
    loss=(math.log(E(1) + E(2) + E(3)) - 3.0 + math.log(3.0)) / 2.0,
    grad=np.array([[0.0450153, 0.1223642, -0.1673795], [-0.3333333, 0.1666667, 0.1666667]], np.float32),
)
CE_SCALED = dict(logits=np.zeros((1, 2), np.float32), targets=np.array([0], np.uint32), scale=1024.0,
                 loss=math.log(2.0), grad=np.array([[-512.0, 512.0]], np.float32))

# tests/linear_backward_test.cu:20-39 (F32 exact small integers, tolerance 1e-5) and :41-53 (F16)
LINEAR_BWD = dict(
    input=np.array([[1, 2, 3], [4, 5, 6]], np.float32),
    weight=np.array([[1, 0, 2], [-1, 3, 1]], np.float32),
    grad_output=np.array([[2, -1], [3, 4]], np.float32),
    grad_input=np.array([[3, -3, 3], [-1, 12, 10]], np.float32),
    grad_weight=np.array([[14, 19, 24], [15, 18, 21]], np.float32),
    grad_bias=np.array([5, 3], np.float32),
)
LINEAR_BWD_F16 = dict(
    input=np.arange(1, 9, dtype=np.float32).reshape(4, 2),
    weight=np.arange(1, 7, dtype=np.float32).reshape(3, 2),
    grad_output=np.arange(1, 13, dtype=np.float32).reshape(4, 3),
    grad_input=np.array([22, 28, 49, 64, 76, 100, 103, 136], np.float32).reshape(4, 2),
    grad_weight=np.array([118, 140, 134, 160, 150, 180], np.float32).reshape(3, 2),
    grad_bias=np.array([22, 26, 30], np.float32),
)

# tests/rope_test.cu:99-127: rotary_dim 2 of head_dim 4, cos/sin rows (1,0) and (0,1); tail copied
ROPE_BWD = dict(
    grad_rotated_query=np.array([1, 2, 30, 40, 3, 4, 50, 60, 5, 6, 70, 80, 7, 8, 90, 100], np.float32).reshape(1, 2, 2, 4),
    grad_rotated_key=np.array([1, -2, 30, 40, 5, -6, 70, 80], np.float32).reshape(1, 2, 1, 4),
    cos=np.array([[1.0], [0.0]], np.float32), sin=np.array([[0.0], [1.0]], np.float32), rotary_dim=2,
    grad_query=np.array([1, 2, 30, 40, 3, 4, 50, 60, 6, -5, 70, 80, 8, -7, 90, 100], np.float32).reshape(1, 2, 2, 4),
    grad_key=np.array([1, -2, 30, 40, -6, -5, 70, 80], np.float32).reshape(1, 2, 1, 4),
)

# tests/embedding_test.cu:183-204: repeated ids accumulate (F16 1e-2, BF16 5e-2)
EMBEDDING_BWD = dict(
    grad_output=np.array([[1, 2, 3, 4], [0.5, 1.5, -1, 2], [7, 8, 9, 10]], np.float32),
    ids=np.array([1, 1, 2], np.uint32), vocab=3,
    grad_weight=np.array([[0, 0, 0, 0], [1.5, 3.5, 2, 6], [7, 8, 9, 10]], np.float32),
)

# tests/adamw_test.cu:21-38: two steps, lr .1, betas .9/.999, eps 1e-8, wd .01 (F32 2e-6, F16 2e-3, BF16 1e-2)
ADAMW_TWO_STEPS = dict(
    parameter=np.array([1.0, -2.0], np.float32), gradient=np.array([0.1, -0.2], np.float32),
    options=dict(learning_rate=0.1, beta1=0.9, beta2=0.999, epsilon=1e-8, weight_decay=0.01),
    after1=np.array([0.899, -1.898], np.float32), m1=np.array([0.01, -0.02], np.float32),
    v1=np.array([0.00001, 0.00004], np.float32), after2=np.array([0.798101, -1.796102], np.float32),
)
# tests/adamw_test.cu:40-58: loss_scale 4, max_grad_norm 1 -> unscaled norm 2 is clipped to 1; then inf is skipped
ADAMW_CLIP = dict(
    parameter=np.array([1.0, -1.0], np.float32), gradient=np.array([8.0, 0.0], np.float32),
    options=dict(learning_rate=0.1, beta1=0.9, beta2=0.999, epsilon=1e-8, weight_decay=0.0, loss_scale=4.0,
                 max_grad_norm=1.0),
    after=np.array([0.9, -1.0], np.float32),
)

# tests/flash_attention_test.cu:306-388: shapes, offsets and scale of the backward cases (tolerance 3e-2,
# inputs there are sin/cos patterns; here seeded normals of the same shapes, checked against the oracle)
ATTENTION_CASES = [
    dict(batch=2, sq=3, sk=5, hq=4, hkv=2, d=32, offset=2, scale=0.23),
    dict(batch=1, sq=3, sk=35, hq=4, hkv=1, d=64, offset=32, scale=0.0),
    dict(batch=1, sq=3, sk=35, hq=4, hkv=1, d=128, offset=32, scale=0.0),
]
