"""The CPU oracle against the committed golden fixtures (tests/golden/*.npz),
which hold what the upstream build produced on seeded inputs.  This is the pin
that travels: it runs where the upstream sources are not available."""
import glob
import os

import numpy as np
import pytest

from oracle import loader

FILES = sorted(f for f in glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz"))
               if "math_known" not in f)


def test_fixture_set_present():
    assert len(FILES) >= 8


@pytest.mark.parametrize("path", FILES, ids=[os.path.basename(f)[:-4] for f in FILES])
def test_oracle_reproduces_golden(orc, path):
    g = np.load(path)
    dim, heads = int(g["dim"]), int(g["heads"])
    for h in range(heads):
        hd = loader.Head(orc, dim, int(g["k_bits"]), int(g["v_bits"]), int(g["capacity"]),
                         loader.mha_head_seed(int(g["base_seed"]), h), float(g["v_mass"]), int(g["hybrid_thresh"]))
        hd.append_many(g["keys"][:, h], g["vals"][:, h])
        assert (hd.k_data() == g[f"k_rows_{h}"]).all()
        assert (hd.v_data() == g[f"v_rows_{h}"]).all()
        assert (hd.k_scale().view(np.uint32) == g[f"k_scale_{h}"].view(np.uint32)).all()
        assert (hd.v_scale().view(np.uint32) == g[f"v_scale_{h}"].view(np.uint32)).all()
        assert (hd.signs() == g[f"signs_{h}"]).all()
        assert [hd.ring_head, hd.size, hd.mirror_tokens] == list(g[f"ring_{h}"])
        for i in range(g["queries"].shape[0]):
            out, n = hd.compute(g["queries"][i, h])
            assert n == hd.size
            assert (out.view(np.uint32) == g["outs"][i, h].view(np.uint32)).all()
