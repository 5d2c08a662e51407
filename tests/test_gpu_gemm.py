"""The hand-written tcgen05 / TMEM / TMA GEMM against a PyTorch fp32 matmul."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def ref(a, b):
    return a.float() @ b.float().t()


# 512: 256 x 256 tiles on CTA pairs (cta_group::2), the ragged last wave split along K; 0: chosen by the cost model
@pytest.mark.parametrize("block_n", [128, 192, 256, 512, 0])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (300, 520, 264), (1, 4096, 4096),
                                   (64, 1792, 4096), (4096, 768, 4096), (1000, 3584, 1024),
                                   (1600, 2800, 1536)])  # 77 pair tiles on 74 pairs: 3 leftover tiles, 6 K ranges each
def test_gemm_matches_fp32(shape, block_n):
    from penny_b200._ext import ops
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    a = (torch.randn(M, K, device="cuda", generator=g) * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda", generator=g) * 0.5).bfloat16()
    out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_bf16(a, b, out, block_n)
    assert ops.gemm_error() == 0
    want = ref(a, b)
    # bf16 output rounding: relative 2^-8 of the value, plus accumulation-order noise
    torch.testing.assert_close(out.float(), want, atol=2e-2 * (K ** 0.5) * 0.25 + 1e-2, rtol=1.6e-2)


def test_gemm_strided_operands_and_repeat():
    from penny_b200._ext import ops
    M, N, K = 512, 384, 320
    big_a = torch.randn(M, K + 64, device="cuda").bfloat16()
    big_b = torch.randn(N, K + 128, device="cuda").bfloat16()
    big_c = torch.zeros(M, N + 32, device="cuda", dtype=torch.bfloat16)
    a, b, c = big_a[:, :K], big_b[:, 64:64 + K], big_c[:, :N]
    for _ in range(3):
        ops.gemm_bf16(a, b, c, 0)
    assert ops.gemm_error() == 0
    torch.testing.assert_close(c.float(), ref(a, b), atol=0.2, rtol=1.6e-2)
    assert torch.all(big_c[:, N:] == 0)


@pytest.mark.parametrize("shape", [(1, 4096, 4096), (64, 1792, 4096), (1600, 2800, 1536), (4096, 3584, 1024)])
def test_gemm_split_tail_repeats(shape):
    """The ragged last wave of the CTA-pair kernel split along K (opt-in): partial
    sums go through a workspace, the last pair to arrive adds them up.  The arrival
    counters live in device memory and reset themselves, so back-to-back launches
    with different operands must each be right."""
    from penny_b200._ext import ops
    M, N, K = shape
    ops.gemm_set_split_tail(1)
    try:
        outs, wants = [], []
        for i in range(3):
            a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
            b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
            out = torch.full((M, N), float("nan"), device="cuda", dtype=torch.bfloat16)
            ops.gemm_bf16(a, b, out, 512)
            outs.append(out)
            wants.append(ref(a, b))
        assert ops.gemm_error() == 0
        for out, want in zip(outs, wants):
            torch.testing.assert_close(out.float(), want, atol=2e-2 * (K ** 0.5) * 0.25 + 1e-2, rtol=1.6e-2)
    finally:
        ops.gemm_set_split_tail(-1)


def test_fused_gemm_kernels_single_rank():
    """GEMM -> reduce-scatter and all-gather -> GEMM with a world of one: the heap
    slots, per-tile flags, the TMA loads from the gathered buffer and the call
    counter all run; only the NVLink hop is missing."""
    from penny_b200._ext import ops
    from penny_b200.parallel.comm import Communicator
    comm = Communicator.emulated(1, heap_bytes=256 << 20, timeout_ms=2000)
    try:
        for it in range(3):  # both scratch halves
            M, N, K = 512, 768, 320
            a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
            w = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
            out = comm.gemm_reduce_scatter(a, w)
            assert ops.gemm_error() == 0
            comm.check()
            torch.testing.assert_close(out.float(), ref(a, w), atol=0.15, rtol=1.6e-2)
            out2 = comm.all_gather_gemm(a, w)
            assert ops.gemm_error() == 0
            comm.check()
            torch.testing.assert_close(out2.float(), ref(a, w), atol=0.15, rtol=1.6e-2)
            N2 = 200  # narrow, ragged N for the gathered variant
            w2 = (torch.randn(N2, K, device="cuda") * 0.5).bfloat16()
            out3 = comm.all_gather_gemm(a, w2, side_ctas=3)
            assert ops.gemm_error() == 0
            torch.testing.assert_close(out3.float(), ref(a, w2), atol=0.15, rtol=1.6e-2)
    finally:
        comm.close()


def test_all_gather_gemm_alternating_shapes_reuse_their_regions():
    """Each (M, K) keeps the gather region it was given on first use: alternating
    two shapes many times must not grow the heap after the first pair."""
    from penny_b200._ext import ops
    from penny_b200.parallel.comm import Communicator
    comm = Communicator.emulated(1, heap_bytes=128 << 20, timeout_ms=2000)
    try:
        shapes = [(256, 320), (384, 192)]
        ws = {K: (torch.randn(128, K, device="cuda") * 0.5).bfloat16() for _, K in shapes}
        free_after_first = None
        for it in range(12):
            for M, K in shapes:
                a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
                out = comm.all_gather_gemm(a, ws[K])
                assert ops.gemm_error() == 0
                comm.check()
                torch.testing.assert_close(out.float(), ref(a, ws[K]), atol=0.15, rtol=1.6e-2)
            if free_after_first is None:
                free_after_first = comm.heap_free()
            assert comm.heap_free() == free_after_first
    finally:
        comm.close()


def test_fused_gemm_kernels_single_rank_cta_pairs():
    """The same two fused kernels on shapes large enough (one 256 x 256 tile per
    CTA pair, K >= 1024) that their launchers choose the cta_group::2 kernel."""
    from penny_b200._ext import ops
    from penny_b200.parallel.comm import Communicator
    comm = Communicator.emulated(1, heap_bytes=512 << 20, timeout_ms=2000)
    try:
        M, N, K = 4096, 1280, 1024
        a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
        w = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
        want = ref(a, w)
        for it in range(3):  # both scratch halves
            out = comm.gemm_reduce_scatter(a, w)
            assert ops.gemm_error() == 0
            comm.check()
            torch.testing.assert_close(out.float(), want, atol=0.3, rtol=1.6e-2)
            out2 = comm.all_gather_gemm(a, w)
            assert ops.gemm_error() == 0
            comm.check()
            torch.testing.assert_close(out2.float(), want, atol=0.3, rtol=1.6e-2)
            out3 = comm.all_gather_gemm(a, w[:768].contiguous())  # 128 x 192 tiles: 128 of them instead of 96
            assert ops.gemm_error() == 0
            comm.check()
            torch.testing.assert_close(out3.float(), want[:, :768], atol=0.3, rtol=1.6e-2)
    finally:
        comm.close()


# ---------------------------------------------------------------------------------------------
# decode GEMM: one CTA per (weight tile, K range), cluster reduction through distributed shared memory
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("splits", [0, 1, 2, 3, 5, 8])
@pytest.mark.parametrize("shape", [(64, 768, 4096), (64, 4096, 512), (7, 1000, 264), (128, 4096, 1024),
                                   (1, 128, 64), (33, 3584, 512), (64, 4096, 1792), (100, 1536, 2048),
                                   (16, 2048, 4096), (8, 16032, 512)])
def test_gemm_decode_matches_fp32(shape, splits):
    """Every cluster size (and the automatic choice), every batch-tile width, ragged N
    and B; called twice in a row with programmatic dependent launch on."""
    from penny_b200._ext import ops
    B, N, K = shape
    if splits > K // 64 and K >= 64:
        pytest.skip("more K ranges than K steps")
    g = torch.Generator(device="cuda").manual_seed(B * 7 + N * 3 + K)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.5).bfloat16()
    for rep in range(2):
        x = (torch.randn(B, K, device="cuda", generator=g) * 0.5).bfloat16()
        out = torch.full((B, N), float("nan"), device="cuda", dtype=torch.bfloat16)
        ops.gemm_decode(x, w, out, False, splits)
        assert ops.gemm_error() == 0
        torch.testing.assert_close(out.float(), ref(x, w), atol=2e-2 * (K ** 0.5) * 0.25 + 1e-2, rtol=1.6e-2)


@pytest.mark.parametrize("splits", [0, 1, 4])
@pytest.mark.parametrize("shape", [(256, 768, 4096), (200, 1000, 512), (129, 4096, 1792), (1024, 256, 128)])
def test_gemm_decode_batch_slabs(shape, splits):
    """Batches above 128 rows: slabs of 128 rows as grid z of one launch (the last one ragged);
    plain and gate/up epilogues."""
    from penny_b200._ext import ops
    B, N, K = shape
    if splits > K // 64:
        pytest.skip("more K ranges than K steps")
    g = torch.Generator(device="cuda").manual_seed(B + N + K)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.5).bfloat16()
    x = (torch.randn(B, K, device="cuda", generator=g) * 0.5).bfloat16()
    out = torch.full((B, N), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_decode(x, w, out, False, splits)
    assert ops.gemm_error() == 0
    torch.testing.assert_close(out.float(), ref(x, w), atol=2e-2 * (K ** 0.5) * 0.25 + 1e-2, rtol=1.6e-2)
    if N % 128 == 0:
        w2 = (w.float() * 0.1).bfloat16()
        out2 = torch.full((B, N // 2), float("nan"), device="cuda", dtype=torch.bfloat16)
        ops.gemm_decode(x, w2, out2, True, splits)
        assert ops.gemm_error() == 0
        y = (x.float() @ w2.float().t()).view(B, N // 128, 2, 64)
        want = (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(B, N // 2)
        torch.testing.assert_close(out2.float(), want, atol=5e-2, rtol=3e-2)


@pytest.mark.parametrize("splits", [0, 1, 4, 7])
@pytest.mark.parametrize("shape", [(64, 3584, 4096), (5, 256, 320), (128, 1792, 1024), (20, 1792, 512)])
def test_gemm_decode_fused_silu_mul(shape, splits):
    """gate/up weight with rows interleaved in blocks of 64: the epilogue returns silu(gate) * up."""
    from penny_b200._ext import ops
    B, F, K = shape
    if splits > K // 64:
        pytest.skip("more K ranges than K steps")
    g = torch.Generator(device="cuda").manual_seed(F + K)
    wg = (torch.randn(F, K, device="cuda", generator=g) * 0.05).bfloat16()
    wu = (torch.randn(F, K, device="cuda", generator=g) * 0.05).bfloat16()
    w = torch.stack([wg.view(F // 64, 64, K), wu.view(F // 64, 64, K)], 1).reshape(2 * F, K).contiguous()
    x = torch.randn(B, K, device="cuda", generator=g).bfloat16()
    out = torch.full((B, F), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.gemm_decode(x, w, out, True, splits)
    assert ops.gemm_error() == 0
    want = torch.nn.functional.silu(x.float() @ wg.float().t()) * (x.float() @ wu.float().t())
    torch.testing.assert_close(out.float(), want, atol=3e-2, rtol=2e-2)


def test_gemm_decode_chain_in_a_cuda_graph_with_and_without_pdl():
    """A chain of dependent decode GEMMs (each reads the previous one's output) captured in a
    CUDA graph: with programmatic dependent launch the kernels overlap their prologues but
    must still see their predecessor's result; the answer equals the serialised run."""
    from penny_b200._ext import ops
    g = torch.Generator(device="cuda").manual_seed(5)
    B, H = 64, 1024
    ws = [(torch.randn(H, H, device="cuda", generator=g) * (1.0 / H ** 0.5)).bfloat16() for _ in range(6)]
    x0 = torch.randn(B, H, device="cuda", generator=g).bfloat16()
    bufs = [torch.empty(B, H, device="cuda", dtype=torch.bfloat16) for _ in range(2)]

    def chain(pdl):
        cur = x0
        for i, w in enumerate(ws):
            ops.gemm_decode(cur, w, bufs[i & 1], False, 0, pdl)
            cur = bufs[i & 1]
        return cur

    want = x0.float()
    for w in ws:
        want = (want @ w.float().t()).bfloat16().float()
    results = {}
    for pdl in (False, True):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            chain(pdl)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = chain(pdl)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        assert ops.gemm_error() == 0
        results[pdl] = out.float().clone()
        torch.testing.assert_close(results[pdl], want, atol=6e-2, rtol=5e-2)
    assert torch.equal(results[False], results[True])
