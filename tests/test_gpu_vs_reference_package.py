"""Device-to-device parity with the reference ITSELF: the unmodified reference package (installed under
baseline/_ref, when present) runs its Triton kernels on the same GPU and the same seeded inputs.
Routing must be identical bit for bit; outputs within max-rel 2e-2; gradients with cosine >= 0.999."""
import os
import subprocess
import sys
import tempfile

import pytest
import torch

from helpers import cos, max_rel
from ref_package_inputs import CASES, make_inputs

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def reference_results():
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "momoe")):
        pytest.skip("reference package not installed under baseline/_ref")
    with tempfile.TemporaryDirectory() as tmp:
        out = os.path.join(tmp, "ref.pt")
        res = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "ref_package_worker.py"), out],
                             capture_output=True, text=True, timeout=900, cwd=ROOT)
        if res.returncode != 0:
            pytest.skip("the reference package did not run here: " + res.stderr[-400:])
        return torch.load(out)


@pytest.mark.parametrize("name", list(CASES))
def test_matches_reference_package_on_device(reference_results, name):
    import __graft_entry__
    __graft_entry__.build()
    import momoe
    from momoe import ops
    assert "momoe-impl_b200" in momoe.__file__
    c, ref = CASES[name], reference_results[name]
    inp = make_inputs(c)
    dev = "cuda"
    moe = momoe.MoE(c["D"], c["H"], c["N"], c["K"], c["Ks"], save_percent=c["sp"], bias_update_rate=1e-3,
                    Wg_DN=inp["Wg"].to(dev), Wl1_ND2H=inp["W1"].to(dev), Wl2_NHD=inp["W2"].to(dev))
    with torch.no_grad():
        moe.biases_N.copy_(inp["biases"].to(dev))
    x = inp["x"].to(dev).requires_grad_(True)
    xo, mask_NM, s_NM = moe.router(x, moe.biases_N)
    y, sizes = moe.momoe(xo, mask_NM, s_NM)
    y.backward(inp["g"].to(dev))
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(mask_NM.cpu(), ref["mask_NM"]), "selected experts differ from the reference's"
    assert torch.equal(sizes.cpu(), ref["sizes"])
    torch.testing.assert_close(s_NM.detach().cpu(), ref["s_NM"], rtol=1e-5, atol=1e-8)
    assert max_rel(y.detach().cpu(), ref["y"]) <= 2e-2
    assert cos(y.detach().cpu(), ref["y"]) >= 0.9999
    for key, got in (("G_x", x.grad), ("G_W1", moe.momoe.Wl1_ND2H.grad), ("G_W2", moe.momoe.Wl2_NHD.grad),
                     ("G_Wg", moe.router.Wg_DN.grad)):
        assert cos(got.cpu(), ref[key]) >= 0.999, "%s cos %g" % (key, cos(got.cpu(), ref[key]))
