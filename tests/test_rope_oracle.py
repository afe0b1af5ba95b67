"""The rotary / KV-scatter oracle against outputs of the reference's own Triton kernels (tests/golden/ref_rope.npz,
made by tests/golden/make_rope_golden.py under Triton's interpreter)."""
import os

import numpy as np
import pytest

from oracle import rope_oracle as rorc
from tests.helpers import ROOT


@pytest.mark.parametrize("name", ["a", "b"])
def test_oracle_against_the_reference_kernels(name):
    g = np.load(os.path.join(ROOT, "tests", "golden", "ref_rope.npz"))
    x, cos, sin = g[f"{name}_x"], g[f"{name}_cos"], g[f"{name}_sin"]
    want = g[f"{name}_rotary"].astype(np.float32)
    got = rorc.rotary_ref(x, cos, sin)
    # the reference multiplies and adds in fp16: up to three roundings of values of magnitude ~|x| apart
    assert np.abs(got - want).max() <= 4e-3 * max(1.0, np.abs(want).max())
    pool = rorc.destindex_copy_ref(g[f"{name}_rotary"], g[f"{name}_dest"], np.full_like(g[f"{name}_pool"], 9.0))
    assert np.array_equal(pool, g[f"{name}_pool"])


def test_rotary_is_a_rotation():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((6, 2, 128)).astype(np.float32)
    ang = rng.uniform(0, 6.28, (6, 64)).astype(np.float32)
    y = rorc.rotary_ref(x, np.cos(ang), np.sin(ang))
    assert np.allclose((y ** 2).sum(-1), (x ** 2).sum(-1), rtol=1e-4)
    assert np.allclose(rorc.rotary_ref(y, np.cos(-ang), np.sin(-ang)), x, atol=1e-4)
    assert np.allclose(rorc.rotary_ref(x.reshape(6, 256), np.cos(ang), np.sin(ang)).reshape(6, 2, 128), y)
