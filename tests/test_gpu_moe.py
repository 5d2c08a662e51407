"""Expert-parallel MoE layer (dispatch + expert FFN + fused combine) with all ranks
emulated on one GPU, against a plain PyTorch fp32 oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4, 8])
def test_moe_layer_emulated(world):
    from penny_b200.models.moe_ep import MoeConfig, MoeEPLayer
    from penny_b200.parallel.comm import Communicator
    comm = Communicator.emulated(world, heap_bytes=256 << 20, timeout_ms=3000)
    try:
        cfg = MoeConfig.tiny()
        T = 96
        layer = MoeEPLayer(cfg, comm, tokens=T, cap_factor=float(world))
        g = torch.Generator(device="cuda").manual_seed(3)
        xs = [torch.randn(T, cfg.hidden, device="cuda", generator=g).bfloat16() for _ in range(world)]
        all_w13 = [layer.w13[e // layer.epr][e % layer.epr] for e in range(cfg.experts)]
        all_w2 = [layer.w2[e // layer.epr][e % layer.epr] for e in range(cfg.experts)]
        want = layer.reference(xs, all_w13, all_w2, layer.router[0])
        for _ in range(2):  # buffers are reused across calls
            outs = layer.forward(xs)
            comm.check()
            for r in range(world):
                torch.testing.assert_close(outs[r].float(), want[r], atol=3e-3, rtol=3e-2)
    finally:
        comm.close()


@pytest.mark.parametrize("shape", [(4096, 8, 2), (1000, 64, 6), (7, 8, 1), (3000, 256, 8)])
def test_device_routing_matches_torch(shape):
    """The routing kernels (top-k + gates, stable counting sort by expert, placement at the owners)
    against the torch formulation they replace."""
    from penny_b200._ext import ops
    from penny_b200.models.moe_ep import build_routing_torch, placement, route_torch
    T, E, K = shape
    g = torch.Generator(device="cuda").manual_seed(T + E)
    # distinct logits per row (a permutation), so top-k has one answer
    perm = torch.rand(T, E, device="cuda", generator=g).argsort(dim=1).float()
    logits = ((perm - E / 2) / 8).bfloat16()
    ids, gates = ops.moe_route(logits, K)
    wi, wg = route_torch(logits, K)
    assert torch.equal(ids, wi)
    torch.testing.assert_close(gates, wg, atol=5e-5, rtol=1e-4)
    order, srt, off, cnt = ops.moe_tables(ids.reshape(-1).contiguous(), E)
    worder, wsrt, woff, wcnt = build_routing_torch(ids, E)
    assert torch.equal(order, worder) and torch.equal(srt, wsrt) and torch.equal(off, woff)
    assert torch.equal(cnt.long(), wcnt)
    for world in (1, 2, 8):
        if E % world:
            continue
        counts_all = torch.randint(0, 50, (world, E), device="cuda", generator=g, dtype=torch.int32)
        dst, rows, ranges = ops.moe_placement(counts_all)
        wdst, wrows, wranges = placement(counts_all.cpu(), world)
        assert torch.equal(dst.cpu(), wdst) and rows.tolist() == wrows
        epr = E // world
        got = [[tuple(ranges[d * epr + le].tolist()) for le in range(epr)] for d in range(world)]
        assert got == wranges
