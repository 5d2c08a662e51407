"""Decode-step kernels and the Llama-shaped decoder against plain PyTorch fp32."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_rope_append_and_attention():
    from penny_b200._ext import ops
    torch.manual_seed(0)
    B, Hq, Hkv, D, L = 5, 8, 2, 128, 300
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    kc = torch.randn(B, Hkv, L, D, device="cuda").bfloat16()
    vc = torch.randn(B, Hkv, L, D, device="cuda").bfloat16()
    pos = torch.tensor([0, 31, 32, 200, 298], dtype=torch.int32, device="cuda")
    q0 = qkv.clone()
    theta = 500000.0
    ops.rope_append(qkv, kc, vc, pos, Hq, Hkv, D, theta)
    # oracle
    inv = theta ** (-torch.arange(0, D // 2, device="cuda", dtype=torch.float32) * 2 / D)
    ang = pos.float()[:, None] * inv[None]
    cos, sin = ang.cos()[:, None], ang.sin()[:, None]

    def rope(t):
        a, b = t[..., :D // 2].float(), t[..., D // 2:].float()
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1)
    q_ref = rope(q0[:, :Hq * D].view(B, Hq, D))
    k_ref = rope(q0[:, Hq * D:(Hq + Hkv) * D].view(B, Hkv, D))
    v_ref = q0[:, (Hq + Hkv) * D:].view(B, Hkv, D)
    torch.testing.assert_close(qkv[:, :Hq * D].view(B, Hq, D).float(), q_ref, atol=3e-2, rtol=2e-2)
    for b in range(B):
        p = int(pos[b])
        torch.testing.assert_close(kc[b, :, p].float(), k_ref[b], atol=3e-2, rtol=2e-2)
        assert torch.equal(vc[b, :, p], v_ref[b])
    for splits in (1, 3, 8):
        out = torch.empty(B, Hq * D, device="cuda", dtype=torch.bfloat16)
        ws = torch.empty(ops.decode_attn_workspace_bytes(B, Hq, splits), dtype=torch.uint8, device="cuda")
        ops.decode_attention(qkv, kc, vc, pos, out, ws, Hq, Hkv, splits, 1.0 / math.sqrt(D))
        G = Hq // Hkv
        for b in range(B):
            p = int(pos[b]) + 1
            q = qkv[b, :Hq * D].view(Hkv, G, D).float()
            s = torch.einsum("hgd,htd->hgt", q, kc[b, :, :p].float()) / math.sqrt(D)
            want = torch.einsum("hgt,htd->hgd", s.softmax(-1), vc[b, :, :p].float()).reshape(Hq * D)
            torch.testing.assert_close(out[b].float(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("pdl", [False, True])
def test_fused_attention_matches_separate_kernels_and_fp32(pdl):
    """rope + KV append + attention + split merge in one launch: same cache rows, same
    output as the three separate kernels and as the fp32 oracle; called twice (the arrival
    counters reset themselves), empty cache included (position 0)."""
    from penny_b200._ext import ops
    torch.manual_seed(3)
    theta = 500000.0
    for B, Hq, Hkv in ((5, 8, 2), (3, 4, 4), (2, 8, 1)):
        D, L = 128, 300
        G = Hq // Hkv
        pos = torch.tensor([0, 31, 32, 200, 298][:B], dtype=torch.int32, device="cuda")
        for splits in (1, 3, 8):
            ws = torch.zeros(ops.decode_attn_fused_workspace_bytes(B, Hq, Hkv, splits), dtype=torch.uint8, device="cuda")
            for rep in range(2):
                qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
                kc = torch.randn(B, Hkv, L, D, device="cuda").bfloat16()
                vc = torch.randn(B, Hkv, L, D, device="cuda").bfloat16()
                # the three-kernel path on copies
                qkv2, kc2, vc2 = qkv.clone(), kc.clone(), vc.clone()
                ops.rope_append(qkv2, kc2, vc2, pos, Hq, Hkv, D, theta)
                out2 = torch.empty(B, Hq * D, device="cuda", dtype=torch.bfloat16)
                ws2 = torch.empty(ops.decode_attn_workspace_bytes(B, Hq, splits), dtype=torch.uint8, device="cuda")
                ops.decode_attention(qkv2, kc2, vc2, pos, out2, ws2, Hq, Hkv, splits, 1.0 / math.sqrt(D))
                # the fused kernel
                out = torch.full((B, Hq * D), float("nan"), device="cuda", dtype=torch.bfloat16)
                ops.decode_attention_fused(qkv, kc, vc, pos, out, ws, Hq, Hkv, splits, 1.0 / math.sqrt(D), theta, pdl)
                torch.cuda.synchronize()
                assert torch.equal(kc, kc2) and torch.equal(vc, vc2)  # same rows appended, nothing else touched
                torch.testing.assert_close(out.float(), out2.float(), atol=2e-2, rtol=2e-2)
                for b in range(B):
                    p = int(pos[b]) + 1
                    q = qkv2[b, :Hq * D].view(Hkv, G, D).float()
                    s = torch.einsum("hgd,htd->hgt", q, kc[b, :, :p].float()) / math.sqrt(D)
                    want = torch.einsum("hgt,htd->hgd", s.softmax(-1), vc[b, :, :p].float()).reshape(Hq * D)
                    torch.testing.assert_close(out[b].float(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("linears", ["penny", "cublas"])
def test_decoder_linears_agree(linears):
    """The decoder on this library's decode GEMM (default) and on cuBLAS produce the same logits."""
    from penny_b200.models.llama_tp import LlamaConfig, LlamaTPDecoder
    cfg = LlamaConfig.tiny()
    m = LlamaTPDecoder(cfg, world=1, max_batch=6, max_len=200, use_graph=True, full_init=True, linears=linears)
    m.fill_synthetic_kv(150)
    m.capture()
    tokens, positions = m.tokens.clone(), m.positions.clone()
    m.step_device()
    torch.cuda.synchronize()
    want = m.reference_logits(tokens, positions, m.kcache, m.vcache)
    err = (m.logits.float() - want).abs().max().item()
    assert err < 0.05 * want.std().item() + 0.02, (linears, err)


def test_decoder_batch_above_128_rows():
    """More than 128 rows: the decode GEMM runs once per 128 rows."""
    from penny_b200.models.llama_tp import LlamaConfig, LlamaTPDecoder
    cfg = LlamaConfig.tiny()
    m = LlamaTPDecoder(cfg, world=1, max_batch=160, max_len=64, use_graph=True, full_init=True)
    m.fill_synthetic_kv(20)
    m.capture()
    tokens, positions = m.tokens.clone(), m.positions.clone()
    m.step_device()
    torch.cuda.synchronize()
    want = m.reference_logits(tokens, positions, m.kcache, m.vcache)
    err = (m.logits.float() - want).abs().max().item()
    assert err < 0.05 * want.std().item() + 0.02, err


def test_silu_mul_and_argmax():
    from penny_b200._ext import ops
    torch.manual_seed(1)
    gu = torch.randn(7, 2 * 1792, device="cuda").bfloat16()
    out = torch.empty(7, 1792, device="cuda", dtype=torch.bfloat16)
    ops.silu_mul(gu, out)
    want = torch.nn.functional.silu(gu[:, :1792].float()) * gu[:, 1792:].float()
    torch.testing.assert_close(out.float(), want, atol=2e-2, rtol=2e-2)
    logits = torch.randn(9, 16032, device="cuda").bfloat16()
    val = torch.empty(9, device="cuda")
    idx = torch.empty(9, dtype=torch.int64, device="cuda")
    ops.argmax_rows(logits, val, idx, 1000)
    wv, wi = logits.float().max(-1)
    assert torch.equal(val, wv)
    # ties: any index holding the max is acceptable, the kernel returns the lowest
    assert torch.equal(logits.float().gather(1, (idx - 1000)[:, None]).squeeze(1), wv)
    # rows cut into chunks (workspace given), ragged and unaligned widths, the (value, index) pair output,
    # twice in a row on the same workspace (the row counters must be back at zero)
    for rows, cols in ((9, 16032), (64, 128256), (3, 1001), (1, 7), (200, 4099)):
        logits = torch.randn(rows, cols, device="cuda").bfloat16()
        logits[0, cols // 2] = 9.0
        logits[0, cols - 1] = 9.0  # a tie: the lower index wins
        ws = torch.zeros(ops.argmax_workspace_bytes(rows), dtype=torch.uint8, device="cuda")
        val = torch.empty(rows, device="cuda")
        idx = torch.empty(rows, dtype=torch.int64, device="cuda")
        pair = torch.empty(2 * rows, device="cuda")
        for _ in range(2):
            ops.argmax_rows(logits, val, idx, 5, ws, pair)
            wv, _ = logits.float().max(-1)
            assert torch.equal(val, wv) and int(idx[0]) == 5 + cols // 2
            assert torch.equal(logits.float().gather(1, (idx - 5)[:, None]).squeeze(1), wv)
            assert torch.equal(pair[:rows], wv) and torch.equal(pair[rows:].long(), idx)
    # the end of a greedy step: best rank per sequence, token fed back, positions advanced
    world, B = 4, 5
    pairs = torch.zeros(world, 2, B, device="cuda")
    pairs[:, 0] = torch.tensor([[1., 5, 2, 0, 3], [4, 5, 1, 0, 2], [0, 1, 9, 0, 3], [2, 2, 2, 0, 8]], device="cuda")
    pairs[:, 1] = torch.arange(world * B, device="cuda").view(world, B).float() + 100
    nxt = torch.zeros(B, dtype=torch.int64, device="cuda")
    tok = torch.zeros(B, dtype=torch.int64, device="cuda")
    pos = torch.full((B,), 7, dtype=torch.int32, device="cuda")
    ops.sample_finish(pairs, world, nxt, tok, pos)
    assert nxt.tolist() == [105, 101, 112, 103, 119] and torch.equal(tok, nxt) and pos.tolist() == [8] * B


@pytest.mark.parametrize("use_graph", [False, True])
def test_decoder_matches_fp32_reference(use_graph):
    from penny_b200.models.llama_tp import LlamaConfig, LlamaTPDecoder
    cfg = LlamaConfig.tiny()
    m = LlamaTPDecoder(cfg, world=1, max_batch=6, max_len=200, use_graph=use_graph, full_init=True)
    m.fill_synthetic_kv(150)
    m.capture()
    tokens, positions = m.tokens.clone(), m.positions.clone()
    m.step_device()
    torch.cuda.synchronize()
    want = m.reference_logits(tokens, positions, m.kcache, m.vcache)
    got = m.logits.float()
    # bf16 pipeline vs fp32 oracle: compare in units of the logit spread
    err = (got - want).abs().max().item()
    assert err < 0.05 * want.std().item() + 0.02, err
    assert torch.equal(m.positions, positions + 1)
    # the chosen token is the (near-)argmax of the reference logits
    chosen = want.gather(1, m.next_tokens[:, None]).squeeze(1)
    assert torch.all(chosen >= want.max(-1).values - 0.1 * want.std())
    # public host API
    host = m.step(torch.zeros(6, dtype=torch.int64))
    assert host.shape == (6,) and host.device.type == "cpu"


def test_sp_prefill_single_rank_matches_fp32():
    """Sequence-parallel prefill block with a world of one: every linear runs the
    fused tcgen05 kernel (heap slots, flags, gathered-buffer TMA), attention,
    RoPE, norms and silu*mul run as in the multi-rank case."""
    from penny_b200.models.llama_sp import LlamaSPPrefill
    from penny_b200.models.llama_tp import LlamaConfig
    from penny_b200.parallel.comm import Communicator
    cfg = LlamaConfig.tiny()
    T, L = 512, 2
    x = torch.randn(T, cfg.hidden, device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)).bfloat16()
    want = LlamaSPPrefill.reference_forward(cfg, x, L, seed=1)
    comm = Communicator.emulated(1, heap_bytes=256 << 20, timeout_ms=2000)
    try:
        for backend in ("penny", "nccl"):
            m = LlamaSPPrefill(cfg, comm=comm, tokens=T, layers=L, backend=backend, seed=1)
            got = m.forward(x).float()
            comm.check()
            rel = ((got - want).norm() / want.norm()).item()
            assert rel < 3e-2, (backend, rel)
    finally:
        comm.close()


def test_rope_rows_matches_reference():
    from penny_b200._ext import ops
    T, Hq, Hkv, D, theta = 37, 4, 2, 128, 500000.0
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    want = qkv.float().clone().view(T, Hq + 2 * Hkv, D)
    half = D // 2
    inv = theta ** (-2.0 * torch.arange(half, device="cuda", dtype=torch.float32) / D)
    ang = (torch.arange(T, device="cuda", dtype=torch.float32) + 11)[:, None] * inv[None]
    c, s_ = ang.cos()[:, None], ang.sin()[:, None]
    a, b = want[:, :Hq + Hkv, :half].clone(), want[:, :Hq + Hkv, half:].clone()
    want[:, :Hq + Hkv, :half] = a * c - b * s_
    want[:, :Hq + Hkv, half:] = b * c + a * s_
    ops.rope_rows(qkv, Hq, Hkv, D, 11, theta)
    torch.testing.assert_close(qkv.float().view(T, Hq + 2 * Hkv, D), want, atol=3e-2, rtol=2e-2)
