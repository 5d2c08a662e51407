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
