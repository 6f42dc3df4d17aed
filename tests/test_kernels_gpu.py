"""Each kernel alone against a plain float32 torch restatement of the same operation, at sizes
other than the engine's: odd widths, tails, head sizes in steps of 16."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _bf16(t):
    return t.to(torch.bfloat16)


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 4096, 2304), (5, 200, 72), (16, 2304, 2048), (33, 1000, 328),
                                   (64, 512, 9216), (100, 130, 8), (256, 256, 256), (300, 384, 520),
                                   (777, 2304, 576),
                                   (2500, 2304, 72),      # 18 x 10 tiles on 148 SMs: token tiles of 240 fill two waves
                                   (3000, 3584, 136)])    # tiles of 256 features, 14 x 14 of them with 224 tokens each
def test_gemm_tcgen05_against_float32(M, N, K):
    from glint_b200 import ops_tensor
    torch.manual_seed(M * 7 + N)
    a = _bf16(torch.randn(M, K, device=DEV))
    w = _bf16(torch.randn(N, K, device=DEV) * 0.1)
    want = a.float() @ w.float().T
    out = torch.full((M, N), float("nan"), device=DEV)
    ops_tensor.gemm(a, w, out, path="tcgen05")
    torch.cuda.synchronize()
    err = (out - want).abs().max().item()
    assert err <= 2e-3 * max(1.0, want.abs().max().item()), (M, N, K, err)


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 4096, 2304), (5, 203, 192), (16, 2304, 2048), (3, 17, 9216),
                                   (9, 1000, 320), (8, 16, 64), (13, 50, 576)])
def test_gemm_skinny_against_float32(M, N, K):
    """The weight-streaming product for a handful of tokens: odd widths, one token, sixteen."""
    from glint_b200 import ops_tensor
    torch.manual_seed(M * 11 + N)
    a = _bf16(torch.randn(M, K, device=DEV))
    w = _bf16(torch.randn(N, K, device=DEV) * 0.1)
    want = a.float() @ w.float().T
    out = torch.full((M, N), float("nan"), device=DEV)
    ops_tensor.gemm(a, w, out, path="skinny")
    again = torch.full((M, N), float("nan"), device=DEV)
    ops_tensor.gemm(a, w, again, path="skinny")
    torch.cuda.synchronize()
    err = (out - want).abs().max().item()
    assert err <= 2e-3 * max(1.0, want.abs().max().item()), (M, N, K, err)
    assert torch.equal(out, again)                                   # the order of the sums is fixed
    # a token's row alone and among others: up to 8 tokens the sums run in the same order (bit for
    # bit); 9 to 16 tokens split K differently among the warps (float32 rounding of the sum)
    alone = torch.empty(1, N, device=DEV)
    ops_tensor.gemm(a[M - 1:].contiguous(), w, alone, path="skinny")
    if M <= 8:
        assert torch.equal(alone[0], out[M - 1])
    else:
        assert (alone[0] - out[M - 1]).abs().max().item() <= 2e-5 * max(1.0, want.abs().max().item())
    out16 = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    ops_tensor.gemm(a, w, out16, cap=30.0, path="skinny")
    capped = 30.0 * torch.tanh(want / 30.0)
    assert (out16.float() - capped).abs().max().item() <= 1e-2 * max(1.0, capped.abs().max().item())


def test_gemm_skinny_refuses_what_it_cannot_do():
    from glint_b200 import ops_tensor
    from glint_b200.errors import KernelError
    a = _bf16(torch.randn(4, 72, device=DEV))
    w = _bf16(torch.randn(32, 72, device=DEV))
    with pytest.raises(KernelError):
        ops_tensor.gemm(a, w, torch.empty(4, 32, device=DEV), path="skinny")       # K is no multiple of 64
    out = torch.empty(4, 32, device=DEV)
    ops_tensor.gemm(a, w, out)                                                     # the tiled kernel takes it
    assert (out - a.float() @ w.float().T).abs().max().item() < 0.05


@pytest.mark.parametrize("features", [300, 7700])
@pytest.mark.parametrize("splits", [1, 2, 3, 7])
def test_gemm_split_k_is_deterministic_and_equal(splits, features):
    """With few tiles every block of a tile adds up a share of its columns; with more tiles than the SMs
    hold at once (7700 features in 3 or 7 splits) the last block to finish adds up all of them."""
    from glint_b200 import ops_tensor
    torch.manual_seed(0)
    a = _bf16(torch.randn(41, 1544, device=DEV))
    w = _bf16(torch.randn(features, 1544, device=DEV) * 0.1)
    want = a.float() @ w.float().T
    outs = []
    for _ in range(3):
        out = torch.empty(41, features, device=DEV)
        ops_tensor.gemm(a, w, out, force_splits=splits, path="tcgen05")
        outs.append(out)
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert (outs[0] - want).abs().max().item() <= 2e-3 * want.abs().max().item()
    one = torch.empty(41, features, device=DEV)
    ops_tensor.gemm(a, w, one, force_splits=1, path="tcgen05")
    assert (outs[0] - one).abs().max().item() <= 1e-5 * want.abs().max().item()


@pytest.mark.parametrize("features", [200, 5000])
@pytest.mark.parametrize("splits", [2, 5])
def test_gated_gemm_split_k(splits, features):
    from glint_b200 import ops_tensor
    torch.manual_seed(1)
    a = _bf16(torch.randn(37, 776, device=DEV))
    w = _bf16(torch.randn(2 * features, 776, device=DEV) * 0.05)
    g, u = a.float() @ w[:features].float().T, a.float() @ w[features:].float().T
    want = torch.nn.functional.gelu(g, approximate="tanh") * u
    outs = []
    for _ in range(2):
        out = torch.empty(37, features, device=DEV, dtype=torch.bfloat16)
        ops_tensor.gemm_gated(a, w, out, "gelu_tanh", force_splits=splits, path="tcgen05")
        outs.append(out)
    assert torch.equal(outs[0], outs[1])
    assert (outs[0].float() - want).abs().max().item() <= 0.01 * want.abs().max().item()


def test_gemm_rows_do_not_depend_on_the_batch():
    from glint_b200 import ops_tensor
    torch.manual_seed(1)
    a = _bf16(torch.randn(70, 1024, device=DEV))
    w = _bf16(torch.randn(2304, 1024, device=DEV) * 0.1)
    whole = torch.empty(70, 2304, device=DEV)
    ops_tensor.gemm(a, w, whole, force_splits=1)
    # rows 0..69 as one launch and in pieces: the K steps are added in an order that depends on the
    # width of the token tile only (1, 2 or 4 interleaved accumulators), so pieces of the same
    # width class agree bit for bit and others to float32 rounding of the sum
    for lo, hi in [(0, 1), (3, 12), (13, 70)]:
        part = torch.empty(hi - lo, 2304, device=DEV)
        ops_tensor.gemm(a[lo:hi].contiguous(), w, part, force_splits=1)
        assert (part - whole[lo:hi]).abs().max().item() <= 2e-5 * whole.abs().max().item(), (lo, hi)
    one = torch.empty(1, 2304, device=DEV)
    nine = torch.empty(9, 2304, device=DEV)
    ops_tensor.gemm(a[5:6].contiguous(), w, one, force_splits=1)
    ops_tensor.gemm(a[3:12].contiguous(), w, nine, force_splits=1)
    assert torch.equal(one[0], nine[2])


def test_gemm_soft_cap_and_bf16_output():
    from glint_b200 import ops_tensor
    torch.manual_seed(2)
    a = _bf16(torch.randn(20, 256, device=DEV))
    w = _bf16(torch.randn(1000, 256, device=DEV))
    want = 30.0 * torch.tanh((a.float() @ w.float().T) / 30.0)
    out = torch.empty(20, 1000, device=DEV)
    ops_tensor.gemm(a, w, out, cap=30.0)
    assert (out - want).abs().max().item() < 5e-3
    out16 = torch.empty(20, 1000, device=DEV, dtype=torch.bfloat16)
    ops_tensor.gemm(a, w, out16, cap=30.0)
    assert (out16.float() - want).abs().max().item() < 0.15


@pytest.mark.parametrize("M,I,K,act", [(7, 320, 96, "gelu_tanh"), (130, 9216, 2304, "gelu_tanh"), (40, 200, 136, "silu"),
                                       (1300, 3840, 72, "gelu_tanh")])     # 30 x 6 tiles: token tiles of 192 instead of 224
def test_gemm_gated_against_float32(M, I, K, act):
    from glint_b200 import ops_tensor
    torch.manual_seed(3)
    a = _bf16(torch.randn(M, K, device=DEV))
    w = _bf16(torch.randn(2 * I, K, device=DEV) * 0.1)
    g, u = a.float() @ w[:I].float().T, a.float() @ w[I:].float().T
    actf = (lambda x: 0.5 * x * (1 + torch.tanh(0.7978846 * (x + 0.044715 * x ** 3)))) if act == "gelu_tanh" \
        else (lambda x: x * torch.sigmoid(x))
    want = actf(g) * u
    out = torch.empty(M, I, device=DEV, dtype=torch.bfloat16)
    ops_tensor.gemm_gated(a, w, out, act, path="tcgen05")
    torch.cuda.synchronize()
    err = (out.float() - want).abs().max().item()
    assert err <= 1e-2 * max(1.0, want.abs().max().item()), err


@pytest.mark.parametrize("M,I,K,act", [(7, 320, 128, "gelu_tanh"), (8, 9216, 2304, "gelu_tanh"), (16, 203, 192, "silu"),
                                       (1, 24, 64, "silu")])
def test_gemm_skinny_gated_against_float32(M, I, K, act):
    from glint_b200 import ops_tensor
    torch.manual_seed(4)
    a = _bf16(torch.randn(M, K, device=DEV))
    w = _bf16(torch.randn(2 * I, K, device=DEV) * 0.1)
    g, u = a.float() @ w[:I].float().T, a.float() @ w[I:].float().T
    actf = (lambda x: 0.5 * x * (1 + torch.tanh(0.7978846 * (x + 0.044715 * x ** 3)))) if act == "gelu_tanh" \
        else (lambda x: x * torch.sigmoid(x))
    want = actf(g) * u
    out = torch.empty(M, I, device=DEV, dtype=torch.bfloat16)
    ops_tensor.gemm_gated(a, w, out, act, path="skinny")
    torch.cuda.synchronize()
    err = (out.float() - want).abs().max().item()
    assert err <= 1e-2 * max(1.0, want.abs().max().item()), err


@pytest.mark.parametrize("M,K,nh,nkv,hd,page,writes", [(8, 2304, 8, 4, 256, 16, True), (3, 192, 5, 1, 48, 32, True),
                                                        (1, 64, 2, 2, 16, 16, True), (7, 320, 6, 3, 80, 16, False),
                                                        (16, 2304, 8, 4, 256, 16, True), (11, 192, 3, 1, 48, 16, True)])
def test_qkv_product_with_rotation_and_cache_write_in_one_kernel(M, K, nh, nkv, hd, page, writes):
    """Against float32 torch: the product, the turn of pairs (j, j + hd/2) by pos * theta^(-2j/hd), and
    the rows of the cache it writes; every other row of the pools stays as it was."""
    from glint_b200 import ops_tensor
    torch.manual_seed(M + hd)
    x = _bf16(torch.randn(M, K, device=DEV))
    w = _bf16(torch.randn((nh + 2 * nkv) * hd, K, device=DEV) * 0.05)
    positions = [37 * i + 5 for i in range(M)]                      # token i of request i
    max_pages = max(positions) // page + 1
    n_pages = M * max_pages + 2
    perm = torch.randperm(n_pages)[:M * max_pages].reshape(M, max_pages).to(torch.int32).to(DEV)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))).to(DEV)
    factor = 2.0
    k_pool = torch.full((n_pages, nkv, page, hd), 7.0, device=DEV, dtype=torch.bfloat16)
    v_pool = torch.full((n_pages, nkv, page, hd), -3.0, device=DEV, dtype=torch.bfloat16)
    q = torch.full((M, nh * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    ops_tensor.qkv_rope(x, w, i32(positions), i32(list(range(M))), perm, inv_freq, factor, q,
                        k_pool if writes else None, v_pool if writes else None, nh, nkv, hd, page, n_pages, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    qkv = (x.float() @ w.float().T).cpu()
    pos = torch.tensor(positions, dtype=torch.float32)
    ang = (pos[:, None] / factor) * inv_freq.cpu()[None, :]          # [M, hd/2]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

    def turn(heads):                                                 # [M, n, hd]
        lo, hi = heads[..., :hd // 2], heads[..., hd // 2:]
        return torch.cat([lo * cos - hi * sin, lo * sin + hi * cos], dim=-1)

    want_q = turn(qkv[:, :nh * hd].reshape(M, nh, hd))
    tol = 2e-2 * max(1.0, qkv.abs().max().item())
    assert (q.float().cpu().reshape(M, nh, hd) - want_q).abs().max().item() <= tol
    if writes:
        want_k = turn(qkv[:, nh * hd:(nh + nkv) * hd].reshape(M, nkv, hd))
        want_v = qkv[:, (nh + nkv) * hd:].reshape(M, nkv, hd)
        kc, vc = k_pool.float().cpu(), v_pool.float().cpu()
        touched = torch.zeros(n_pages, page, dtype=torch.bool)
        for t, p_ in enumerate(positions):
            pg = int(perm[t, p_ // page])
            assert (kc[pg, :, p_ % page] - want_k[t]).abs().max().item() <= tol
            assert (vc[pg, :, p_ % page] - want_v[t]).abs().max().item() <= tol
            touched[pg, p_ % page] = True
        assert (kc.permute(0, 2, 1, 3)[~touched] == 7.0).all() and (vc.permute(0, 2, 1, 3)[~touched] == -3.0).all()
    else:
        assert (k_pool == 7.0).all() and (v_pool == -3.0).all()


@pytest.mark.parametrize("lens,starts,K,nh,nkv,hd,page,writes,min_blocks", [
    ([300, 41, 2], [0, 77, 1000], 136, 3, 1, 256, 16, True, 0),    # three requests, 343 tokens: two token tiles
    ([300, 41, 2], [0, 77, 1000], 136, 3, 1, 256, 16, True, 12),   # tiles of 128 tokens to have 12 blocks
    ([5], [3], 64, 2, 2, 512, 32, True, 0),                         # two groups of 128 pairs per head
    ([600], [4090], 2304, 8, 4, 256, 16, True, 0),
    ([2400, 100], [0, 7], 72, 8, 4, 256, 16, True, 0),             # 16 x 10 tiles on 148 SMs: token tiles of 240
    ([70, 9], [0, 5], 200, 1, 1, 256, 16, False, 0)])
def test_tiled_qkv_product_with_rotation_and_cache_write(lens, starts, K, nh, nkv, hd, page, writes, min_blocks):
    """The same on the tiled kernel for portions of prompts: the angles come from a table made by
    ``rope_table``; tokens of one request share its row of the block table."""
    from glint_b200 import ops, ops_tensor
    torch.manual_seed(sum(lens) + hd)
    M = sum(lens)
    x = _bf16(torch.randn(M, K, device=DEV))
    w = _bf16(torch.randn((nh + 2 * nkv) * hd, K, device=DEV) * 0.05)
    positions = [s + i for n, s in zip(lens, starts) for i in range(n)]
    seq = [r for r, n in enumerate(lens) for _ in range(n)]
    max_pages = max(positions) // page + 1
    n_pages = len(lens) * max_pages + 2
    perm = torch.randperm(n_pages)[:len(lens) * max_pages].reshape(len(lens), max_pages).to(torch.int32).to(DEV)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, hd, 2, dtype=torch.float32) / hd))).to(DEV)
    factor = 1.0 if hd == 256 else 4.0
    k_pool = torch.full((n_pages, nkv, page, hd), 7.0, device=DEV, dtype=torch.bfloat16)
    v_pool = torch.full((n_pages, nkv, page, hd), -3.0, device=DEV, dtype=torch.bfloat16)
    q = torch.full((M, nh * hd), float("nan"), device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    trig = torch.empty(M, hd // 2, 2, device=DEV)
    ops.rope_table(i32(positions), inv_freq, factor, trig)
    pos = torch.tensor(positions, dtype=torch.float32)
    ang = (pos[:, None] / factor) * inv_freq.cpu()[None, :]          # [M, hd/2]
    assert (trig[..., 0].cpu() - torch.cos(ang)).abs().max().item() < 1e-3     # float32 angles up to 4000 rad
    assert (trig[..., 1].cpu() - torch.sin(ang)).abs().max().item() < 1e-3
    assert ops_tensor.qkv_rope_tiled_supported(M, K, hd, hd, nh + 2 * nkv, min_blocks=min_blocks)
    assert not ops_tensor.qkv_rope_tiled_supported(M, K, hd, hd, nh + 2 * nkv, min_blocks=10 ** 6)
    ops_tensor.qkv_rope_tiled(x, w, trig, i32(positions), i32(seq), perm, q, k_pool if writes else None,
                              v_pool if writes else None, nh, nkv, hd, page, n_pages, status, min_blocks=min_blocks)
    torch.cuda.synchronize()
    assert status.item() == 0
    qkv = (x.float() @ w.float().T).cpu()
    cos, sin = trig[..., 0].cpu()[:, None, :], trig[..., 1].cpu()[:, None, :]

    def turn(heads):                                                 # [M, n, hd]
        lo, hi = heads[..., :hd // 2], heads[..., hd // 2:]
        return torch.cat([lo * cos - hi * sin, lo * sin + hi * cos], dim=-1)

    want_q = turn(qkv[:, :nh * hd].reshape(M, nh, hd))
    tol = 1e-2 * max(1.0, qkv.abs().max().item())
    assert (q.float().cpu().reshape(M, nh, hd) - want_q).abs().max().item() <= tol
    if writes:
        want_k = turn(qkv[:, nh * hd:(nh + nkv) * hd].reshape(M, nkv, hd))
        want_v = qkv[:, (nh + nkv) * hd:].reshape(M, nkv, hd)
        kc, vc = k_pool.float().cpu(), v_pool.float().cpu()
        rows = torch.tensor([int(perm[r, p_ // page]) for r, p_ in zip(seq, positions)])
        slots = torch.tensor([p_ % page for p_ in positions])
        assert (kc[rows, :, slots] - want_k).abs().max().item() <= tol
        assert (vc[rows, :, slots] - want_v).abs().max().item() <= tol
        touched = torch.zeros(n_pages, page, dtype=torch.bool)
        touched[rows, slots] = True
        assert (kc.permute(0, 2, 1, 3)[~touched] == 7.0).all() and (vc.permute(0, 2, 1, 3)[~touched] == -3.0).all()
    else:
        assert (k_pool == 7.0).all() and (v_pool == -3.0).all()


# ---- attention over a paged cache -----------------------------------------------------------------

def _paged_case(seq_lens_before, seq_lens_new, nkv, hd, page_size, dtype, seed, hot=None, v_poison=float("nan")):
    """Random keys/values for every request laid into shuffled pages.  Returns the pools, the block
    table [requests, max_pages], and the dense per-request K, V [len, nkv, hd]."""
    g = torch.Generator().manual_seed(seed)
    totals = [a + b for a, b in zip(seq_lens_before, seq_lens_new)]
    max_pages = max(-(-t // page_size) for t in totals) + 1
    n_pages = sum(-(-t // page_size) for t in totals) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    k_pool = torch.full((n_pages, nkv, page_size, hd), float("nan"))
    v_pool = torch.full((n_pages, nkv, page_size, hd), v_poison)
    table = torch.full((len(totals), max_pages), -1, dtype=torch.int32)
    dense = []
    for s, total in enumerate(totals):
        k = torch.randn(total, nkv, hd, generator=g).to(dtype).float()
        v = torch.randn(total, nkv, hd, generator=g).to(dtype).float()
        if hot is not None and hot[0] == s:      # one far key that must win the softmax
            k[hot[1]] *= 6.0
        dense.append((k, v))
        for p in range(-(-total // page_size)):
            page = perm.pop()
            table[s, p] = page
            lo, hi = p * page_size, min(total, (p + 1) * page_size)
            k_pool[page, :, :hi - lo] = k[lo:hi].transpose(0, 1)
            v_pool[page, :, :hi - lo] = v[lo:hi].transpose(0, 1)
    return k_pool.to(dtype).to(DEV), v_pool.to(dtype).to(DEV), table.to(DEV), dense


def _attention_reference(q, dense, seq_of_token, positions, nh, nkv, multiplier, cap, window):
    out = torch.zeros_like(q)
    G = nh // nkv
    for t in range(q.shape[0]):
        k, v = dense[seq_of_token[t]]
        pos = positions[t]
        lo = max(0, pos - window + 1) if window else 0
        for h in range(nh):
            s = (k[lo:pos + 1, h // G] @ q[t, h]) * multiplier
            if cap:
                s = cap * torch.tanh(s / cap)
            out[t, h] = torch.softmax(s, 0) @ v[lo:pos + 1, h // G]
    return out


def _stream_attention(qd, k_pool, v_pool, positions, seq_of_token, table, out, nh, nkv, hd, page, mult, cap, window,
                      status, blocks, arrive=None, pair_cost=-1):
    """The single-token kernel that shares all pages of the launch evenly among ``blocks`` blocks."""
    from glint_b200 import ops_tensor
    T = positions.shape[0]
    plan = ops_tensor.attention_decode_stream_plan(positions, seq_of_token, T, window, page, hd, nkv, blocks, min_pages=1,
                                                   pair_cost=pair_cost)
    partials = torch.full((ops_tensor.stream_workspace_floats(blocks, nh, nkv, hd),), float("nan"), dtype=torch.float32,
                          device=DEV)
    arrive = torch.zeros(T * nkv, dtype=torch.int32, device=DEV) if arrive is None else arrive
    ops_tensor.attention_decode_stream(qd, k_pool, v_pool, positions, seq_of_token, table, out, nh, nkv, hd, page,
                                       k_pool.shape[0], mult, cap, window, status, plan, partials, arrive)
    assert int(arrive.abs().sum().item()) == 0, "the arrival counters are not back at zero"
    pages_per_block, pages = plan[1].cpu().tolist()
    return pages_per_block, pages


ATT_CASES = [
    # nh, nkv, hd, page, before,            new,             window, cap
    (8, 4, 256, 16, [300, 0, 1023, 77], [1, 1, 1, 1], None, 50.0),
    (8, 4, 256, 16, [300, 0, 1023, 77], [1, 1, 1, 1], 128, 50.0),
    (6, 1, 32, 16, [0, 40, 5], [33, 2, 70], 8, 20.0),
    (6, 2, 48, 16, [10, 0, 200], [50, 129, 1], 40, None),
    (4, 2, 16, 16, [0, 17], [64, 3], 16, 50.0),
    (32, 16, 128, 16, [500, 0], [1, 130], 100, 30.0),
    (3, 3, 80, 32, [90], [45], None, 10.0),
    (16, 1, 64, 16, [31], [20], None, None),
    (4, 2, 256, 64, [100, 3], [1, 1], None, 50.0),          # pages of 64 at head size 256: three stages, not four
]


@pytest.mark.parametrize("kernel", ["plain32", "plain16", "decode", "stream", "prefill", "tcgen05"])
@pytest.mark.parametrize("case", range(len(ATT_CASES)))
def test_attention_kernels_against_float32(case, kernel):
    from glint_b200 import ops, ops_tensor
    nh, nkv, hd, page, before, new, window, cap = ATT_CASES[case]
    if kernel == "stream" and nh // nkv > 8:
        pytest.skip("more than 8 query heads per kv head: the cluster kernel takes it")
    if kernel == "prefill" and not ops_tensor.prefill_supported(nh, nkv, hd):
        pytest.skip("size outside the tiled kernel's range (the split kernel takes it)")
    if kernel == "tcgen05" and not ops_tensor.tcgen05_attention_supported(nh, nkv, hd, page):
        pytest.skip("size outside the tcgen05 kernel's range")
    dtype = torch.float32 if kernel == "plain32" else torch.bfloat16
    # the tcgen05 kernel multiplies masked keys' values by exactly zero: its poison must be finite
    k_pool, v_pool, table, dense = _paged_case(before, new, nkv, hd, page, dtype, seed=case,
                                               v_poison=3.0e4 if kernel == "tcgen05" else float("nan"))
    seq_of_token, positions = [], []
    for s, (b, n) in enumerate(zip(before, new)):
        seq_of_token += [s] * n
        positions += list(range(b, b + n))
    T = len(positions)
    torch.manual_seed(case)
    q = (torch.randn(T, nh, hd) * 1.5).to(dtype)
    mult = 1.0 / math.sqrt(hd)
    want = _attention_reference(q.float(), dense, seq_of_token, positions, nh, nkv, mult, cap, window)
    qd = q.reshape(T, nh * hd).to(DEV)
    out = torch.full_like(qd, float("nan"))
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    if kernel.startswith("plain"):
        ops.attention_plain(qd, k_pool, v_pool, i32(positions), i32(seq_of_token), table, out, nh, nkv, hd, page,
                            k_pool.shape[0], mult, cap, window, status)
    elif kernel == "decode":
        for splits in (1, 3):
            ops_tensor.attention_decode(qd, k_pool, v_pool, i32(positions), i32(seq_of_token), table, out, nh, nkv,
                                        hd, page, k_pool.shape[0], mult, cap, window, status, splits)
            got = out.float().cpu().reshape(T, nh, hd)
            assert (got - want).abs().max().item() < 0.03, splits
    elif kernel == "stream":
        # one block for everything; blocks that end inside pairs; more blocks than pages (a page per block)
        arrive = torch.zeros(T * nkv, dtype=torch.int32, device=DEV)
        for blocks, pair_cost in ((1, -1), (5, 0), (5, 3), (37, 1), (37, -1), (2000, 0), (2000, 2)):
            out.fill_(float("nan"))
            per_block, units = _stream_attention(qd, k_pool, v_pool, i32(positions), i32(seq_of_token), table, out, nh,
                                                 nkv, hd, page, mult, cap, window, status, blocks, arrive, pair_cost)
            assert per_block == max(1, -(-units // blocks))
            got = out.float().cpu().reshape(T, nh, hd)
            assert (got - want).abs().max().item() < 0.03, blocks
    else:
        cu = [0]
        for n in new:
            cu.append(cu[-1] + n)
        fn = ops_tensor.attention_prefill if kernel == "prefill" else ops_tensor.attention_tcgen05
        fn(qd, k_pool, v_pool, i32(cu), i32(before), table, out, len(new), max(new), nh, nkv, hd, page,
           k_pool.shape[0], mult, cap, window, status)
    got = out.float().cpu().reshape(T, nh, hd)
    assert int(status.item()) == 0
    tol = 2e-5 if kernel == "plain32" else 0.03
    assert (got - want).abs().max().item() < tol, (got - want).abs().max().item()


def test_single_token_attention_says_which_pages_it_takes():
    from glint_b200 import ops_tensor
    assert ops_tensor.decode_supported(8, 4, 256, 16) and ops_tensor.decode_supported(8, 4, 256, 64)
    assert not ops_tensor.decode_supported(8, 4, 256, 128)       # three stages of such pages do not fit an SM
    assert ops_tensor.decode_supported(32, 16, 128, 128) and ops_tensor.decode_supported(4, 1, 64, 256)
    assert not ops_tensor.decode_supported(8, 3, 256, 16) and not ops_tensor.decode_supported(8, 4, 24, 16)


@pytest.mark.parametrize("kernel", ["plain16", "decode", "stream", "prefill", "tcgen05"])
def test_attention_finds_one_far_key_among_hundreds(kernel):
    """One key far back is scaled so that its score stands out: the output must be its value row."""
    from glint_b200 import ops, ops_tensor
    nh, nkv, hd, page = 8, 4, 256, 16
    before, new = [900], [1]
    hot_pos = 37
    k_pool, v_pool, table, dense = _paged_case(before, new, nkv, hd, page, torch.bfloat16, seed=9,
                                               v_poison=3.0e4 if kernel == "tcgen05" else float("nan"))
    k, v = dense[0]
    q = torch.zeros(1, nh, hd)
    for h in range(nh):
        q[0, h] = k[hot_pos, h // 2] * 4.0          # aligned with the far key: its score dominates
    q = q.to(torch.bfloat16)
    want = _attention_reference(q.float(), dense, [0], [900], nh, nkv, 1 / 16.0, None, None)
    assert (want[0, 0] - v[hot_pos, 0]).abs().max() < 1e-2       # the case does what it says
    qd = q.reshape(1, nh * hd).to(DEV)
    out = torch.empty_like(qd)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    if kernel == "plain16":
        ops.attention_plain(qd, k_pool, v_pool, i32([900]), i32([0]), table, out, nh, nkv, hd, page, k_pool.shape[0],
                            1 / 16.0, None, None, status)
    elif kernel == "decode":
        ops_tensor.attention_decode(qd, k_pool, v_pool, i32([900]), i32([0]), table, out, nh, nkv, hd, page,
                                    k_pool.shape[0], 1 / 16.0, None, None, status, 7)
    elif kernel == "stream":
        _stream_attention(qd, k_pool, v_pool, i32([900]), i32([0]), table, out, nh, nkv, hd, page, 1 / 16.0, None, None,
                          status, 23)
    else:
        fn = ops_tensor.attention_prefill if kernel == "prefill" else ops_tensor.attention_tcgen05
        fn(qd, k_pool, v_pool, i32([0, 1]), i32([900]), table, out, 1, 1, nh, nkv, hd, page, k_pool.shape[0], 1 / 16.0,
           None, None, status)
    got = out.float().cpu().reshape(1, nh, hd)
    assert (got - want).abs().max().item() < 0.03


@pytest.mark.parametrize("kernel", ["plain16", "decode", "stream", "prefill", "tcgen05"])
@pytest.mark.parametrize("pos", [63, 64, 79, 80, 200])
def test_attention_window_edge(kernel, pos):
    """A hot key just outside the window must not be seen; the same key just inside must win.
    Positions put the window's edge on, before and after a page boundary."""
    from glint_b200 import ops, ops_tensor
    nh, nkv, hd, page, window = 4, 2, 64, 16, 33
    for inside in (False, True):
        hot = pos - window + 1 if inside else pos - window
        k_pool, v_pool, table, dense = _paged_case([pos], [1], nkv, hd, page, torch.bfloat16, seed=pos, hot=None,
                                                   v_poison=3.0e4 if kernel == "tcgen05" else float("nan"))
        k, v = dense[0]
        q = torch.zeros(1, nh, hd)
        for h in range(nh):
            q[0, h] = k[hot, h // 2] * 3.0
        q = q.to(torch.bfloat16)
        want = _attention_reference(q.float(), dense, [0], [pos], nh, nkv, 0.125, None, window)
        near_hot = (want[0, 0] - v[hot, 0]).abs().max().item()
        assert (near_hot < 0.05) == inside                   # the case separates the two outcomes
        qd = q.reshape(1, nh * hd).to(DEV)
        out = torch.empty_like(qd)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
        if kernel == "plain16":
            ops.attention_plain(qd, k_pool, v_pool, i32([pos]), i32([0]), table, out, nh, nkv, hd, page,
                                k_pool.shape[0], 0.125, None, window, status)
        elif kernel == "decode":
            ops_tensor.attention_decode(qd, k_pool, v_pool, i32([pos]), i32([0]), table, out, nh, nkv, hd, page,
                                        k_pool.shape[0], 0.125, None, window, status, 2)
        elif kernel == "stream":
            _stream_attention(qd, k_pool, v_pool, i32([pos]), i32([0]), table, out, nh, nkv, hd, page, 0.125, None,
                              window, status, 3)
        else:
            fn = ops_tensor.attention_prefill if kernel == "prefill" else ops_tensor.attention_tcgen05
            fn(qd, k_pool, v_pool, i32([0, 1]), i32([pos]), table, out, 1, 1, nh, nkv, hd, page, k_pool.shape[0],
               0.125, None, window, status)
        got = out.float().cpu().reshape(1, nh, hd)
        assert (got - want).abs().max().item() < 0.03, (inside, (got - want).abs().max().item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,H", [(1, 64), (5, 96), (3, 2304), (2, 1002), (4, 10000)])
def test_norm_kernels_against_float32(rows, H, dtype):
    from glint_b200 import ops
    torch.manual_seed(H)
    x = torch.randn(rows, H, device=DEV) * 3
    y = torch.randn(rows, H, device=DEV)
    wa, wb = torch.randn(H, device=DEV) * 0.2, torch.randn(H, device=DEV) * 0.2
    norm = lambda t, w, eps, off: t * torch.rsqrt((t * t).mean(-1, keepdim=True) + eps) * (off + w)
    out = torch.empty(rows, H, device=DEV, dtype=dtype)
    ops.rmsnorm(x, wa, out, 1e-6, 1.0)
    tol = 1e-5 if dtype == torch.float32 else 0.05
    assert (out.float() - norm(x, wa, 1e-6, 1.0)).abs().max().item() < tol
    idx = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, H, device=DEV, dtype=dtype)
    ops.rmsnorm(x, wa, out2, 1e-5, 0.0, idx)
    assert (out2.float() - norm(x[[rows - 1, 0]], wa, 1e-5, 0.0)).abs().max().item() < tol
    x2 = x.clone()
    ops.add_rmsnorm(x2, y, (wa, 1e-6, 1.0), out, (wb, 1e-5, 1.0))
    want_x = x + norm(y, wa, 1e-6, 1.0)
    assert (x2 - want_x).abs().max().item() < 1e-5
    assert (out.float() - norm(want_x, wb, 1e-5, 1.0)).abs().max().item() < tol
    x3 = x.clone()
    ops.add_rmsnorm(x3, y, None, None, None)
    assert torch.equal(x3, x + y)


@pytest.mark.parametrize("V", [512, 1000, 256000, 777])
def test_argmax_takes_the_last_maximum(V):
    from glint_b200 import ops
    torch.manual_seed(V)
    logits = torch.randn(3, V, device=DEV)
    logits[1, 5] = logits[1, V - 3] = 99.0          # equal maxima: the later index wins
    logits[2, 0] = 50.0
    out = torch.empty(3, dtype=torch.int32, device=DEV)
    ops.argmax(logits, out)
    assert out.tolist() == [int(torch.argmax(logits[0])), V - 3, 0]


@pytest.mark.parametrize("V", [32768, 256000, 100003])
def test_argmax_of_wide_rows_by_several_blocks(V):
    """Rows shared by several blocks: equal maxima in different chunks, -0 against +0, a row of
    -inf, twice in a row (the per-row scratch is left zeroed); with an odd width the rows start at
    every alignment."""
    from glint_b200 import ops
    torch.manual_seed(V)
    logits = torch.randn(5, V, device=DEV)
    logits[1, 7] = logits[1, V - 2] = logits[1, V // 2] = 77.0
    logits[2].fill_(-1.0)
    logits[2, 3] = 0.0
    logits[2, V - 5] = -0.0                                # equal to +0: the later index wins
    logits[3].fill_(float("-inf"))
    logits[4, 0] = 1e30
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    for _ in range(2):
        out.fill_(-7)
        ops.argmax(logits, out)
        assert out.tolist() == [int(torch.argmax(logits[0])), V - 2, V - 5, V - 1, 0]


def test_sampling_kernel_against_the_plain_sampler():
    from glint_b200 import ops
    from tests.plain import sampler as ps
    V = 1000
    g = torch.Generator().manual_seed(0)
    cases = [dict(temperature=0.8), dict(temperature=1.0), dict(temperature=1.3, top_k=20),
             dict(temperature=0.7, top_p=0.9), dict(temperature=1.0, min_p=0.05),
             dict(temperature=0.9, top_k=50, top_p=0.8, min_p=0.01)]
    agree = total = 0
    for ci, opts in enumerate(cases):
        for trial in range(12):
            logits = (torch.randn(V, generator=g) * 2.5).float()
            rng_a, rng_b = ps.Xorshift64(100 * ci + trial), ps.Xorshift64(100 * ci + trial)
            want = ps.sample(logits.numpy(), [], rng_a, **opts)
            u = float(rng_b.next_f32())
            dev = lambda v, dt: torch.tensor([v], dtype=dt, device=DEV)
            out = torch.empty(1, dtype=torch.int32, device=DEV)
            work = torch.empty(1, V, device=DEV)
            ops.sample(logits.to(DEV).view(1, V), work, dev(opts["temperature"], torch.float32),
                       dev(opts.get("top_k", 0), torch.int32), dev(opts.get("top_p", 1.0), torch.float32),
                       dev(opts.get("min_p", 0.0), torch.float32), dev(u, torch.float32), out)
            agree += int(out.item() == want)
            total += 1
    # sums are added in another order on the device: a draw that lands within rounding of a
    # boundary of the cumulative distribution may fall to the neighbour
    assert agree >= total - 2, (agree, total)


def _exact_distribution(logits, past, temperature=1.0, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0):
    """The sampler's stages in float64 (tests/plain/sampler.py in higher precision; top-k keeps every
    element equal to the k-th, as the device does): the final probabilities."""
    x = np.asarray(logits, dtype=np.float64).copy()
    for t in past:
        x[t] = x[t] / repeat_penalty if x[t] > 0 else x[t] * repeat_penalty
    x = x / temperature
    if 0 < top_k < len(x):
        kth = np.sort(x)[-top_k]
        x[x < kth] = -np.inf
    if min_p > 0.0:
        x[x < x.max() + np.log(min_p)] = -np.inf
    p = np.exp(x - x.max())
    p /= p.sum()
    if top_p < 1.0:
        order = np.argsort(-p, kind="stable")
        cut = int(np.searchsorted(np.cumsum(p[order]), top_p, side="left")) + 1
        kept = np.zeros_like(p)
        kept[order[:cut]] = p[order[:cut]]
        p = kept / kept.sum()
    return p


@pytest.mark.parametrize("V", [16384, 100003, 256000])
def test_sampling_of_wide_rows_by_a_cluster(V):
    """Rows of 16 K entries and more are shared by the blocks of a cluster.  Peaked rows must give the
    plain sampler's token; on flat rows, where thousands of tokens share the mass and 32-bit running sums
    differ in their last digits, the token must be the one whose interval of the exact cumulative
    distribution holds the draw, to within 1e-3 of mass.  All rows of a case go in one launch."""
    from glint_b200 import ops
    from tests.plain import sampler as ps
    g = torch.Generator().manual_seed(V)
    cases = [dict(temperature=0.8), dict(temperature=1.0, top_k=40), dict(temperature=0.7, top_p=0.9),
             dict(temperature=1.0, min_p=0.05), dict(temperature=0.9, top_k=50, top_p=0.8, min_p=0.01),
             dict(temperature=1.3, top_k=1), dict(temperature=1.0, top_p=0.3, repeat_penalty=1.7),
             dict(temperature=0.6, top_k=2000, top_p=0.95, repeat_penalty=1.2)]
    for spread, exact in ((9.0, True), (2.0, False)):
        rows = len(cases)
        logits = (torch.randn(rows, V, generator=g) * spread).float()
        logits[1, 77] = logits[1, V - 5] = logits[1].max() + 1.0          # equal values at the top
        pasts = [[] if "repeat_penalty" not in c else
                 [int(t) for t in torch.topk(logits[i], 6).indices.tolist()] * 2 + [3, V - 1, 3]
                 for i, c in enumerate(cases)]
        us = [float(ps.Xorshift64(1000 * V + i).next_f32()) for i in range(rows)]
        f32 = lambda v: torch.tensor(v, dtype=torch.float32, device=DEV)
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        offsets, toks, counts = [0], [], []
        for past in pasts:
            uniq = sorted(set(past))
            toks += uniq
            counts += [past.count(t) for t in uniq]
            offsets.append(len(toks))
        out = torch.full((rows,), -1, dtype=torch.int32, device=DEV)
        work = torch.empty(rows, V, device=DEV)
        dev_logits = logits.to(DEV)
        args = (dev_logits, work, f32([c["temperature"] for c in cases]), i32([c.get("top_k", 0) for c in cases]),
                f32([c.get("top_p", 1.0) for c in cases]), f32([c.get("min_p", 0.0) for c in cases]), f32(us), out)
        pens = (i32(offsets), i32(toks), i32(counts), f32([c.get("repeat_penalty", 1.0) for c in cases]))
        ops.sample_rows(*args, penalties=pens)
        got = out.tolist()
        out.fill_(-1)
        ops.sample_rows(*args, penalties=pens)
        assert out.tolist() == got                                         # the same twice
        assert torch.equal(dev_logits.cpu(), logits)                       # the logits are left as they were
        agree = 0
        for i, c in enumerate(cases):
            p = _exact_distribution(logits[i].numpy(), pasts[i], **c)
            cdf = np.cumsum(p)
            j = got[i]
            assert 0 <= j < V and p[j] > 0, (V, spread, i, j)
            assert cdf[j] - p[j] - 1e-3 <= us[i] < cdf[j] + 1e-3, (V, spread, i, j, us[i], cdf[j] - p[j], cdf[j])
            if exact:
                class _U:                                                   # the plain sampler draws the same u
                    def next_f32(self, u=us[i]):
                        return np.float32(u)
                agree += int(ps.sample(logits[i].numpy(), pasts[i], _U(), **c) == j)
        if exact:
            assert agree >= rows - 1, (V, agree)
        assert got[5] == int(torch.argmax(logits[5]))                      # top_k = 1


@pytest.mark.parametrize("V", [16384, 100003, 256000])
def test_sampling_of_wide_rows_at_the_edges(V):
    """Rows that leave the usual paths of the cluster kernel: equal logits everywhere (every element is a
    tie at the threshold; thousands of candidates in one bin), one finite logit, none, one dominant
    logit, two equal maxima under top_k = 1, a tiny temperature, a large top-k."""
    from glint_b200 import ops

    def run(logits, temp=1.0, k=0, p=1.0, mp=0.0, u=0.5):
        rows = logits.shape[0]
        f32 = lambda v: torch.full((rows,), v, dtype=torch.float32, device=DEV)
        out = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
        ops.sample_rows(logits.to(DEV).contiguous(), torch.empty(rows, V, device=DEV), f32(temp),
                        torch.full((rows,), k, dtype=torch.int32, device=DEV), f32(p), f32(mp), f32(u), out)
        return out.tolist()

    near = lambda want: (lambda g: abs(g - want) <= max(2, V // 2000))
    flat = torch.zeros(2, V)
    assert all(map(near(V // 2), run(flat, u=0.5)))
    assert all(map(near(V // 4), run(flat, k=10, u=0.25)))                 # ties at the k-th value are all kept
    assert all(map(near(V), run(flat, p=0.5, u=0.9999)))                   # and at the top-p boundary
    one = torch.full((2, V), float("-inf"))
    one[:, V - 3] = 1.0
    assert run(one, k=5, p=0.9, u=0.7) == [V - 3, V - 3]
    assert all(map(near(V // 2), run(torch.full((2, V), float("-inf")), u=0.5)))   # nothing finite: uniform
    torch.manual_seed(V)
    dom = torch.randn(2, V)
    dom[:, 77] = 60.0
    assert run(dom, temp=0.7, p=0.9, u=0.9999) == [77, 77]
    two = torch.randn(2, V)
    two[:, 5] = two[:, V - 9] = 30.0
    assert run(two, k=1, u=0.4) == [5, 5] and run(two, k=1, u=0.6) == [V - 9, V - 9]
    spread = torch.randn(2, V) * 3
    assert run(spread, temp=1e-3, u=0.3) == spread.argmax(1).tolist()
    kth = torch.topk(spread, 3000, dim=1).values[:, -1]
    got = run(spread, k=3000, u=0.99999)
    assert all(spread[r, g] >= kth[r] for r, g in enumerate(got)), got


def test_repeat_penalty_kernel():
    from glint_b200 import ops
    V = 64
    logits = torch.tensor([[2.0] * V, [-1.0] * V], device=DEV)
    work = torch.empty(2, V, device=DEV)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    ops.apply_penalty(logits, work, i32([0, 2, 3]), i32([5, 9, 7]), i32([3, 1, 2]),
                      torch.tensor([2.0, 1.5], device=DEV))
    assert work[0, 5].item() == 0.25 and work[0, 9].item() == 1.0 and work[0, 0].item() == 2.0
    assert work[1, 7].item() == pytest.approx(-2.25) and work[1, 5].item() == -1.0


def test_runtime_routes_products_by_size():
    """Which product kernel the native runtime takes: the weight-streaming one up to 8 tokens, and from 9 to
    16 for small matrices; the tiled one beyond; neither when K is no multiple of 8 (CUDA cores then)."""
    from glint_b200 import ops_tensor
    assert ops_tensor.route_linear(1, 4096, 2304) == 1 and ops_tensor.route_linear(8, 9216, 2304) == 1
    assert ops_tensor.route_linear(8, 36864, 4608) == 2            # the widest matrices stream on the tiled kernel
    assert ops_tensor.route_linear(16, 2304, 2048) == 1            # 9 to 16 tokens, a small matrix
    assert ops_tensor.route_linear(16, 9216, 2304) == 2            # 9 to 16 tokens, a large one
    assert ops_tensor.route_linear(17, 2304, 2048) == 2 and ops_tensor.route_linear(2048, 4096, 2304) == 2
    assert ops_tensor.route_linear(4, 256000, 2304) == 2           # the output head streams on the tiled kernel
    assert ops_tensor.route_linear(4, 4096, 2296) == 2             # K in steps of 8 but not of 64
    assert ops_tensor.route_linear(4, 4096, 2300) == 0
    assert ops_tensor.decode_splits(1, 4, 8192, 148) == 16 and ops_tensor.decode_splits(8, 4, 2304, 148) == 8
    assert ops_tensor.decode_splits(64, 4, 2304, 148) == 1 and ops_tensor.decode_splits(8, 4, 200, 148) == 1
    assert ops_tensor.decode_splits(9, 4, 2304, 148) == 4          # 36 clusters of 8 would not fit the SMs at once
    # contexts that add up to half of (requests x longest): the longest is shared among more blocks
    assert ops_tensor.decode_splits(56, 4, 8192, 148) == 1 and ops_tensor.decode_splits(56, 4, 8192, 148, uneven=1) == 4
    assert ops_tensor.decode_splits(56, 8, 8192, 148, uneven=1) == 2 and ops_tensor.decode_splits(12, 4, 8192, 148, uneven=1) == 8
    assert ops_tensor.decode_splits(64, 4, 300, 148, uneven=1) == 2   # never fewer than 128 keys to a split
    assert ops_tensor.decode_splits(8, 4, 2304, 148, uneven=2) == 8   # and never fewer splits than even contexts get
    assert ops_tensor.decode_splits(9, 8, 2304, 148) == 2          # 72 clusters of 4 do not fit either
    # the kernel that shares all pages of a launch evenly: uneven contexts from 32 (token, kv head) pairs, even ones
    # where the clusters would leave SMs idle or single blocks make more than a wave
    streams = lambda t, nkv, uneven=0, nh=None: ops_tensor.decode_streams(t, nh or 2 * nkv, nkv, 4096, 148, uneven)
    assert not streams(8, 4) and streams(9, 4) and not streams(16, 4) and not streams(64, 4) and streams(64, 8)
    assert streams(12, 4) and streams(24, 4) and streams(48, 4) and streams(4, 4) and not streams(1, 4)
    assert streams(56, 4, 1) and streams(8, 4, 1) and not streams(7, 4, 1) and streams(9, 8) and not streams(8, 8)
    assert not streams(64, 4, 1, nh=64)                            # 16 query heads per kv head: the cluster kernel
