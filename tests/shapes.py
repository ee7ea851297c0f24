"""Problem shapes used across the tests.

``REFERENCE_TEST_SHAPES`` follows the categories of the reference's own test parameters
(tests/test_conv2d_gw8.py:67-180): all 25 filter sizes, zero / large / asymmetric padding,
1..16 groups, odd extents, and its named regression cases.  ``MODEL_SHAPES`` is a sample of
the real-model layer shapes the reference keeps in spio/src_tests/Conv2dGw8Params.dat with
the batch reduced so that the CPU oracle finishes in seconds.
"""

from oracle.oracle import Shape

# (shape, has_bias)
SANITY = [
    (Shape(4, 64, 16, 32, 3, 3, 1, 1), True),
    (Shape(4, 48, 32, 32, 3, 3, 1, 1), False),
    (Shape(1, 64, 8, 16, 3, 3, 1, 1), False),
    (Shape(4, 128, 32, 32, 4, 1, 2, 0), True),       # functional grad sanity: 4x1 filter, pad (2,0)
    (Shape(2, 1632, 10, 10, 5, 5, 2, 2), True),      # wgrad resource regression (n reduced from 64)
]

FILTER_SIZES = [
    (Shape(1, 128, 32, 32, r, s, r // 2, s // 2), (r + s) % 2 == 0)
    for r in range(1, 6) for s in range(1, 6)
]

PADDING = [
    (Shape(1, 128, 64, 64, 3, 3, 0, 0), False),
    (Shape(4, 128, 20, 19, 3, 3, 0, 0), True),
    (Shape(1, 128, 64, 64, 3, 3, 2, 2), False),
    (Shape(1, 128, 64, 64, 3, 3, 7, 7), True),
]

GROUPS = [(Shape(4, 8 * g, 32, 32, 3, 3, 1, 1), g % 2 == 0) for g in range(1, 17)]

MISC = [
    (Shape(6, 128, 49, 33, 3, 3, 1, 1), True),
    (Shape(6, 128, 6, 5, 3, 3, 1, 1), False),
    (Shape(16, 1024, 7, 7, 3, 3, 1, 1), True),
    (Shape(8, 64, 64, 64, 3, 3, 1, 1), False),
    (Shape(3, 128, 16, 16, 3, 3, 1, 1), True),
    (Shape(4, 128, 32, 16, 3, 3, 1, 1), False),
    (Shape(5, 128, 16, 32, 3, 3, 1, 1), True),
    (Shape(6, 128, 48, 32, 3, 3, 1, 1), False),
]

def load_model_shapes(max_batch: int = 0):
    """The 81 real-model layer shapes of the reference (spio/src_tests/Conv2dGw8Params.dat), from the
    fixture tests/golden/model_shapes.json that tests/golden/make_golden.py writes; ``max_batch``
    caps the batch so that the CPU oracle finishes in seconds."""
    import json
    from pathlib import Path

    rows = json.loads((Path(__file__).resolve().parent / "golden" / "model_shapes.json").read_text())
    return [(Shape(min(d["n"], max_batch) if max_batch else d["n"], d["c"], d["h"], d["w"], d["r"], d["s"],
                   d["pad_h"], d["pad_w"]), bool(d["has_bias"])) for d in rows]


MODEL_SHAPES = [
    (Shape(4, 80, 56, 56, 5, 5, 2, 2), True),
    (Shape(4, 160, 28, 28, 5, 5, 2, 2), True),
    (Shape(8, 320, 14, 14, 5, 5, 2, 2), True),
    (Shape(8, 640, 7, 7, 5, 5, 2, 2), True),
    (Shape(8, 1248, 8, 8, 3, 3, 1, 1), False),
    (Shape(8, 1392, 9, 9, 5, 5, 2, 2), False),
    (Shape(2, 144, 64, 64, 3, 3, 1, 1), False),
    (Shape(1, 16, 128, 128, 3, 3, 1, 1), False),
    (Shape(2, 192, 72, 72, 3, 3, 1, 1), False),
    (Shape(1, 24, 144, 144, 3, 3, 1, 1), False),
    (Shape(4, 256, 28, 28, 3, 3, 1, 1), True),
    (Shape(2, 288, 36, 36, 5, 5, 2, 2), False),
    (Shape(1, 40, 144, 144, 3, 3, 1, 1), False),
    (Shape(8, 512, 14, 14, 3, 3, 1, 1), True),
    (Shape(4, 576, 18, 18, 5, 5, 2, 2), False),
    (Shape(8, 1152, 7, 7, 5, 5, 2, 2), False),
]

# The configurations the headline metric is quoted on (batch reduced where noted by tests).
CFG1 = Shape(8, 64, 32, 32, 3, 3, 1, 1)
CFG2 = lambda n: Shape(n, 64, 56, 56, 3, 3, 1, 1)  # noqa: E731
CFG3 = [(128, 56), (256, 28), (512, 14), (768, 7)]
CFG4 = [(96, 56), (192, 28), (384, 14), (768, 7)]

REFERENCE_TEST_SHAPES = SANITY + FILTER_SIZES + PADDING + GROUPS + MISC + MODEL_SHAPES


def ident(case) -> str:
    sh, bias = case
    return (f"n{sh.n}c{sh.c}h{sh.h}w{sh.w}r{sh.r}s{sh.s}p{sh.pad_h}x{sh.pad_w}" + ("b" if bias else ""))
