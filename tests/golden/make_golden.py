"""Generates the golden fixtures in this folder by running the UNMODIFIED reference kernels on CPU.

Run where a checkout of the reference is available, with REFERENCE_ROOT pointing at it:

    REFERENCE_ROOT=<reference checkout> python tests/golden/make_golden.py

The reference's Triton kernels execute under `TRITON_INTERPRET=1`.  Three shims touch Triton (not the
reference): every autotuner is pinned to one of its own configurations (it cannot benchmark without a
GPU); the interpreter's `dot` converts bf16 operands to fp32 before multiplying (Triton 3.6's
interpreter multiplies the raw uint16 bit patterns otherwise); and the interpreter's fp32->bf16 cast, which
truncates, is replaced by round-to-nearest-even, the conversion Triton emits on a GPU.  The `MoE` wrapper hard-codes "cuda", so the
script composes TopKRouter -> MoMoE -> bias update exactly as momoe/sample_moe.py:59-68 does.

Each case is stored as `<name>.npz`; bf16 tensors are stored as their uint16 bit patterns (`*_bf16`).
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
sys.dont_write_bytecode = True
REF = os.environ.get("REFERENCE_ROOT")
if not REF or not os.path.isdir(os.path.join(REF, "momoe")):
    sys.exit("set REFERENCE_ROOT to a checkout of the reference repository (the folder that contains momoe/)")
sys.path.insert(0, REF)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton.language as tl  # noqa: E402
import triton.runtime.interpreter as ti  # noqa: E402
from triton.runtime.autotuner import Autotuner  # noqa: E402


def _dot(self, a, b, d, input_precision, max_num_imprecise_acc):
    ad, bd = a.data, b.data
    if a.dtype.scalar == tl.bfloat16:
        ad = ti._convert_float(ad, tl.bfloat16, tl.float32, None).view(np.float32).reshape(a.data.shape)
    if b.dtype.scalar == tl.bfloat16:
        bd = ti._convert_float(bd, tl.bfloat16, tl.float32, None).view(np.float32).reshape(b.data.shape)
    return ti.TensorHandle(np.matmul(ad, bd, dtype=d.data.dtype) + d.data, d.dtype.scalar)


ti.InterpreterBuilder.create_dot = _dot

_orig_convert = ti._convert_float


def _convert_rne(inp, input_dtype, output_dtype, rounding_mode):
    if input_dtype == tl.float32 and output_dtype == tl.bfloat16:
        u = np.ascontiguousarray(inp).view(np.uint32).astype(np.uint64)
        rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
        nan = np.isnan(np.ascontiguousarray(inp).view(np.float32))
        rounded[nan.reshape(rounded.shape)] = 0x7FC0
        return rounded.reshape(inp.shape)
    return _orig_convert(inp, input_dtype, output_dtype, rounding_mode)


ti._convert_float = _convert_rne

import momoe.momoe as ref_momoe  # noqa: E402
from momoe.topk_router import TopKRouter  # noqa: E402

_ORIG_CONFIGS = {}
for _n in dir(ref_momoe):
    _k = getattr(ref_momoe, _n)
    if isinstance(_k, Autotuner):
        _ORIG_CONFIGS[_n] = list(_k.configs)


def pin_tile_config(i):
    for n, cfgs in _ORIG_CONFIGS.items():
        getattr(ref_momoe, n).configs = [cfgs[min(i, len(cfgs) - 1)]]


def bits(t):
    return t.detach().contiguous().view(torch.int16).numpy().view(np.uint16)


def run_case(name, B, S, D, H, N, K, Ks, save_percent, tile_cfg, block_rows, bias_std, seed, w_std=0.02):
    pin_tile_config(tile_cfg)
    torch.manual_seed(seed)
    M = B * S
    x0 = torch.randn(B, S, D)
    W1 = (torch.randn(N, D, 2 * H) * w_std).bfloat16()
    W2 = (torch.randn(N, H, D) * w_std).bfloat16()
    Wg = (torch.randn(D, N) * w_std).bfloat16()
    biases = torch.cat([torch.randn(N - Ks) * bias_std, torch.full((Ks,), float("-inf"))])

    # (A) whole chain: router -> experts -> loss -> backward (momoe/sample_moe.py:59-68)
    router = TopKRouter(D, N, K, Ks, Wg_DN=Wg)
    moe = ref_momoe.MoMoE(D, H, N, K, save_percent=save_percent, Wl1_ND2H=W1, Wl2_NHD=W2)
    x = x0.clone().requires_grad_(True)
    xo, mask_NM, s_NM = router(x, biases)
    y, sizes = moe(xo, mask_NM, s_NM)
    c_avg = M * (K - Ks) / (N - Ks)
    new_biases = biases + 1e-4 * torch.sign(c_avg - sizes)
    (y.float() ** 2).sum().backward()

    cumsums, idx, counts, which = ref_momoe.find_used_experts(mask_NM, K)

    # (B) experts only with leaf x and s: isolates G_s and the experts' own G_x
    moe_b = ref_momoe.MoMoE(D, H, N, K, save_percent=save_percent, Wl1_ND2H=W1, Wl2_NHD=W2)
    xb = x0.bfloat16().clone().requires_grad_(True)
    sb = s_NM.detach().clone().requires_grad_(True)
    yb, _ = moe_b(xb, mask_NM, sb)
    (yb.float() ** 2).sum().backward()

    out = dict(
        meta=np.array([B, S, D, H, N, K, Ks, block_rows], dtype=np.int64),
        save_percent=np.array(save_percent, dtype=np.float64),
        x=x0.numpy(), W1_bf16=bits(W1), W2_bf16=bits(W2), Wg_bf16=bits(Wg), biases=biases.numpy(),
        mask_NM=mask_NM.numpy(), s_NM=s_NM.detach().contiguous().numpy(), sizes=sizes.numpy(),
        cumsums=cumsums.numpy(), idx=idx.numpy(), which=which.numpy(),
        y_bf16=bits(y), new_biases=new_biases.numpy(),
        G_x=x.grad.numpy(), G_W1_bf16=bits(moe.Wl1_ND2H.grad), G_W2_bf16=bits(moe.Wl2_NHD.grad),
        G_Wg_bf16=bits(router.Wg_DN.grad),
        G_s_NM=sb.grad.numpy(), G_x_experts_bf16=bits(xb.grad),
    )
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), name + ".npz")
    np.savez_compressed(path, **out)
    print(name, "sizes", sizes.tolist(), "->", path, os.path.getsize(path) // 1024, "KiB")


if __name__ == "__main__":
    # the reference's CPU-runnable configuration: D256 H128 N8 K2, x fp32 [2,64,256], save_percent 0, seed 0
    run_case("cfg1_d256_h128_n8_k2", 2, 64, 256, 128, 8, 2, 0, 0, tile_cfg=0, block_rows=128,
             bias_std=0.0, seed=0)
    # shared expert + biased router + save_percent cutting through the expert-major order (128-row tiles)
    run_case("shared_d64_h32_n6_k3_ks1_sp50", 1, 96, 64, 32, 6, 3, 1, 50, tile_cfg=0, block_rows=128,
             bias_std=0.05, seed=1)
    # 64-row tiles, save_percent 50: saved and recomputed tiles inside one expert
    run_case("tiles64_d64_h64_n4_k2_sp50", 1, 512, 64, 64, 4, 2, 0, 50, tile_cfg=2, block_rows=64,
             bias_std=0.0, seed=2)
    # everything saved
    run_case("sp100_d128_h64_n4_k2", 2, 48, 128, 64, 4, 2, 0, 100, tile_cfg=0, block_rows=128,
             bias_std=0.02, seed=3)
    # 24 tokens, 16 experts, strong bias: all tokens land on two experts, fourteen experts receive nothing
    run_case("empty_experts_d128_h64_n16_k2", 1, 24, 128, 64, 16, 2, 0, 0, tile_cfg=0, block_rows=128,
             bias_std=0.5, seed=4)
    # two shared experts, K = 5, H not a multiple of 64, save_percent 30
    run_case("shared2_d128_h96_n12_k5_ks2_sp30", 1, 80, 128, 96, 12, 5, 2, 30, tile_cfg=0, block_rows=128,
             bias_std=0.05, seed=5)
    # top-8 of 32 experts on 64 tokens: a realistic K with several experts without tokens
    run_case("top8_d128_h64_n32_k8", 1, 64, 128, 64, 32, 8, 0, 0, tile_cfg=0, block_rows=128,
             bias_std=0.02, seed=6)
    # save_percent 99 with 64-row tiles: only the last rows of the last expert are recomputed
    run_case("sp99_d64_h64_n4_k2_tiles64", 1, 300, 64, 64, 4, 2, 0, 99, tile_cfg=2, block_rows=64,
             bias_std=0.0, seed=7)
