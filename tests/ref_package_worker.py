"""Runs the UNMODIFIED reference package (pip-installed under baseline/_ref) on seeded inputs on the GPU and saves what
it produced.  Launched as a subprocess by test_gpu_vs_reference_package.py because its package name, `momoe`, is the
same as this repository's drop-in package."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main(out_path):
    import momoe as ref
    from ref_package_inputs import CASES, make_inputs
    assert "baseline" in ref.__file__
    results = {}
    for name, c in CASES.items():
        inp = make_inputs(c)
        dev = "cuda"
        moe = ref.MoE(c["D"], c["H"], c["N"], c["K"], c["Ks"], save_percent=c["sp"], bias_update_rate=1e-3,
                      Wg_DN=inp["Wg"].to(dev), Wl1_ND2H=inp["W1"].to(dev), Wl2_NHD=inp["W2"].to(dev))
        with torch.no_grad():
            moe.biases_N.copy_(inp["biases"].to(dev))
        x = inp["x"].to(dev).requires_grad_(True)
        # same composition as MoE.forward, unrolled to expose the routing tensors
        xo, mask_NM, s_NM = moe.router(x, moe.biases_N)
        y, sizes = moe.momoe(xo, mask_NM, s_NM)
        y.backward(inp["g"].to(dev))
        torch.cuda.synchronize()
        results[name] = dict(mask_NM=mask_NM.cpu(), s_NM=s_NM.detach().cpu().contiguous(), sizes=sizes.cpu(),
                             y=y.detach().cpu(), G_x=x.grad.cpu(), G_W1=moe.momoe.Wl1_ND2H.grad.cpu(),
                             G_W2=moe.momoe.Wl2_NHD.grad.cpu(), G_Wg=moe.router.Wg_DN.grad.cpu())
    torch.save(results, out_path)


if __name__ == "__main__":
    main(sys.argv[1])
