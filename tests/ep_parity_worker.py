"""Worker of the multi-GPU expert-parallel parity test (launched by torchrun, one rank per GPU).

Every rank builds the same seeded global problem, runs (a) the single-GPU `MoE` on ALL tokens with ALL experts and
(b) `ExpertParallelMoE` on its own token shard with its own expert block, and compares: y and dX of its shard,
dW of its expert block, the summed gate gradient, the global tokens_per_expert and the bias update."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "momoe-impl_b200"))
sys.path.insert(0, os.path.join(ROOT, "tests"))


def run_case(transport, case, rank, world, dev, momoe, ep, ops, cos, max_rel):
    Mr, D, H, N, K, Ks, sp, bias_std = case
    g = torch.Generator().manual_seed(1234 + D)
    x_all = torch.randn(world, 1, Mr, D, generator=g).bfloat16()
    W1 = (torch.randn(N, D, 2 * H, generator=g) * 0.03).bfloat16()
    W2 = (torch.randn(N, H, D, generator=g) * 0.03).bfloat16()
    Wg = (torch.randn(D, N, generator=g) * 0.05).bfloat16()
    gy_all = torch.randn(world, 1, Mr, D, generator=g).bfloat16()
    biases = torch.cat([torch.randn(N - Ks, generator=g) * bias_std, torch.full((Ks,), float("-inf"))])
    Nl = N // world
    # (a) single GPU, all tokens
    ref = momoe.MoE(D, H, N, K, Ks, save_percent=sp, bias_update_rate=1e-3, Wg_DN=Wg.to(dev),
                    Wl1_ND2H=W1.to(dev), Wl2_NHD=W2.to(dev))
    with torch.no_grad():
        ref.biases_N.copy_(biases.to(dev))
    # (b) expert parallel, own shard
    # the sharded layer starts from other weights and takes the single-GPU layer's checkpoint with a plain
    # load_state_dict: keys as in the reference, every rank keeps its own block of the [N, ...] expert tensors
    moe = ep.ExpertParallelMoE(D, H, N, K, Ks, save_percent=sp, bias_update_rate=1e-3,
                               Wg_DN=torch.zeros(D, N, device=dev), Wl1_ND2H=torch.zeros(Nl, D, 2 * H, device=dev),
                               Wl2_NHD=torch.zeros(Nl, H, D, device=dev), transport=transport.split("-")[0],
                               capacity_factor=float(world))   # room for any routing, however skewed
    # "peer": transfers and GEMMs of the forward pass in sequence; "peer-halves": the local experts in two halves whose
    # transfers overlap the other half's GEMMs (what large passes do by default)
    moe.forward_chunks = 2 if transport == "peer-halves" else 1
    ckpt = {k: v.detach().clone() for k, v in ref.state_dict().items()}
    res = moe.load_state_dict(ckpt)
    assert not res.missing_keys and not res.unexpected_keys
    assert torch.equal(moe.Wl1_ND2H, W1[rank * Nl:(rank + 1) * Nl].to(dev))
    assert torch.equal(moe.biases_N, biases.to(dev))
    xa = x_all.reshape(1, world * Mr, D).to(dev).requires_grad_(True)
    ya = ref(xa)
    ya.backward(gy_all.reshape(1, world * Mr, D).to(dev))
    xr = x_all[rank].to(dev).requires_grad_(True)
    yr = moe(xr)
    yr.backward(gy_all[rank].to(dev))
    torch.cuda.synchronize()
    ops.check_status(dev)
    sl = slice(rank * Mr, (rank + 1) * Mr)
    assert torch.equal(moe.biases_N, ref.biases_N), "bias update (global tokens_per_expert) differs"
    # same kernels, same per-row arithmetic: y rows are identical bits
    assert torch.equal(yr[0], ya[0, sl]), "y differs: max-rel %g" % max_rel(yr[0], ya[0, sl])
    assert cos(xr.grad[0], xa.grad[0, sl]) > 0.9999 and max_rel(xr.grad[0], xa.grad[0, sl]) < 2e-2
    for name, got, full in (("W1", moe.Wl1_ND2H.grad, ref.momoe.Wl1_ND2H.grad),
                            ("W2", moe.Wl2_NHD.grad, ref.momoe.Wl2_NHD.grad)):
        want = full[rank * Nl:(rank + 1) * Nl]
        assert cos(got, want) > 0.9999, name
        assert max_rel(got, want) < 2e-2, name
    gwg = moe.router.Wg_DN.grad.float().clone()
    dist.all_reduce(gwg)
    assert cos(gwg, ref.router.Wg_DN.grad) > 0.999
    if rank == 0:
        print("ep parity ok:", transport, (Mr, D, H, N, K, Ks, sp), "world", world, flush=True)


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import momoe
    from momoe import ep, ops
    from helpers import cos, max_rel

    cases = [  # tokens per rank, D, H, N, K, Ks, save_percent, bias_std
        (192, 256, 128, 8, 2, 0, 0, 0.0),
        (1000, 512, 256, 16, 4, 0, 50, 0.05),
        (512, 384, 136, 8, 3, 1, 100, 0.02),
    ]
    for transport in ("peer", "peer-halves", "nccl"):
        for case in cases:
            run_case(transport, case, rank, world, dev, momoe, ep, ops, cos, max_rel)
    # buffers far too small for the routing: every rank must notice (device status 302) and nothing may fault
    g = torch.Generator().manual_seed(77)
    D, H, K = 256, 128, 2
    N = 2 * world
    moe = ep.ExpertParallelMoE(D, H, N, K, 0, Wg_DN=(torch.randn(D, N, generator=g) * 0.05).bfloat16().to(dev),
                               Wl1_ND2H=torch.zeros(N // world, D, 2 * H, device=dev),
                               Wl2_NHD=torch.zeros(N // world, H, D, device=dev), capacity_factor=0.05)
    moe.forward_chunks = 2
    x = torch.randn(1, 4096, D, generator=g).bfloat16().to(dev).requires_grad_(True)
    moe(x).sum().backward()
    torch.cuda.synchronize()
    # nobody calls check_status: the next forward pass of the layer must raise by itself
    try:
        moe(x)
        raise AssertionError("overflow of the expert-parallel buffers was not reported")
    except RuntimeError as err:
        assert "302" in str(err), err
    torch.cuda.synchronize()
    ops.check_status(dev)          # reported once, then cleared
    if rank == 0:
        print("ep overflow reported ok", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
