"""The Nulalorn design in the engine against its plain restatement (``plain_nulalorn``): each mechanism alone, whole
prompts, token-by-token decoding, portions, batches of unequal requests, slots and pages used again, far keys, page
borders and window edges, the first tokens, long decoding past the ring of a windowed cache, sizes of one, and
greedy generation through ``generate`` and the command line.

float32 is compared strictly.  bfloat16 is compared by the error of a row relative to the row's size: the choice of
experts is a table look-up, so no row can go another way than the plain implementation's, and every row is held."""

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import ondeviceinfer_b200 as odi
import plain_nulalorn as plain
from helpers import assert_logits_close, write_model_folder
from ondeviceinfer_b200.kernels import ops
from ondeviceinfer_b200.parts.linear import flush_residual_add

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
CONFIGS = {"A": (plain.TINY_A, 31), "B": (plain.TINY_B, 32), "C": (plain.TINY_C, 33), "sharp": (plain.SHARP, 34),
           "bare": (plain.PLAIN_STACK, 35), "wide": (plain.WIDE_HEADS, 36)}
_MODELS, _PLAIN = {}, {}


def weights_of(case):
    return plain.random_weights(*CONFIGS[case])


def engine(case, dtype, tmp_path_factory):
    if (case, dtype) not in _MODELS:
        folder = write_model_folder(tmp_path_factory.mktemp(f"nulalorn_{case}"), CONFIGS[case][0], weights_of(case))
        _MODELS[(case, dtype)] = odi.load_resident_model(folder, dtype=dtype)
    return _MODELS[(case, dtype)]


def expected(case, tokens):
    key = (case, tuple(tokens))
    if key not in _PLAIN:
        _PLAIN[key] = plain.forward(CONFIGS[case][0], weights_of(case), list(tokens))[0].float()
    return _PLAIN[key]


def close(actual, reference, dtype, what):
    """float32: the helpers' strict comparison.  bfloat16: row error relative to the row's size: median at most
    1.5e-2, nine rows in ten within 5e-2, every row within 1.5e-1 (a row of small logits has a large relative error)."""
    if dtype == "float32":
        assert_logits_close(actual, reference, dtype, what)
        return
    actual, reference = actual.float().cpu(), reference.float().cpu()
    assert actual.shape == reference.shape and torch.isfinite(actual).all(), what
    error = (actual - reference).norm(dim=-1) / reference.norm(dim=-1).clamp_min(1e-6)
    ranked = error.sort().values
    high = ranked[int(0.9 * len(ranked))] if len(ranked) >= 10 else ranked[-1]
    assert float(ranked[-1]) <= 1.5e-1 and float(error.median()) <= 1.5e-2 and float(high) <= 5e-2, \
        f"{what}: bfloat16 row errors median {float(error.median()):.3e}, high {float(high):.3e}, max {float(ranked[-1]):.3e}"


# ----------------------------------------------------------------------------- kernels against plain functions


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,dv,rot,nq,nkv", [(16, 8, 8, 4, 2), (6, 5, 6, 3, 1), (96, 40, 2, 2, 2), (36, 36, 0, 1, 1), (160, 24, 160, 2, 1)])
def test_head_preparation_rotates_then_norms(dtype, d, dv, rot, nq, nkv):
    g = torch.Generator().manual_seed(d)
    n, eps, lanes = 70, 1e-3, -(-d // 4) * 4
    qkv = torch.randn(n, (nq + nkv) * d + nkv * dv, generator=g).to(dtype)
    pos = torch.randint(0, 500, (n,), generator=g).int()
    freqs = plain.rotary_frequencies(rot, 50.0) if rot else None
    q_out = torch.full((n, nq * lanes), 7.0, dtype=dtype, device="cuda")
    k_pool = torch.zeros((n, nkv, 64, lanes), dtype=dtype, device="cuda")       # a ring of one page per token
    v_pool = torch.zeros((n, nkv, 64, dv), dtype=dtype, device="cuda")
    cos = sin = None
    if rot:
        angle = pos.double()[:, None] * freqs[None, :]
        cos, sin = torch.cos(angle).float().cuda(), torch.sin(angle).float().cuda()
    seq = torch.arange(n, dtype=torch.int32, device="cuda")
    ops.rot_unit_prep(qkv.cuda(), q_out, k_pool, v_pool, cos, sin, seq, pos.cuda(), seq, seq, nq=nq, nkv=nkv, d=d, dv=dv,
                      rot_dim=rot, page_size=64, ring_pages=1, write_kv=True, unit_eps=eps, d_store=lanes)
    wide = qkv.double()
    q, k = wide[:, :nq * d].view(n, nq, d), wide[:, nq * d:(nq + nkv) * d].view(n, nkv, d)
    if rot:
        q, k = plain.rotate_pairs(q, pos, freqs), plain.rotate_pairs(k, pos, freqs)
    q, k = plain.rms_norm(q, None, eps), plain.rms_norm(k, None, eps)
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    got_q = q_out.view(n, nq, lanes).cpu().double()
    rows = torch.arange(n)
    got_k = k_pool[rows, :, (pos % 64).long()].cpu().double()
    assert (got_q[..., :d] - q).abs().max() < tol and (got_k[..., :d] - k).abs().max() < tol
    assert float(got_q[..., d:].abs().sum()) == 0 and float(got_k[..., d:].abs().sum()) == 0
    assert torch.equal(v_pool[rows, :, (pos % 64).long()].cpu().view(n, -1), qkv[:, (nq + nkv) * d:])


def _paged(x, n_pages):
    """[T, heads, lanes] -> pool [pages, heads, 64, lanes] with position p in page p // 64."""
    T, heads, lanes = x.shape
    pool = torch.zeros((n_pages, heads, 64, lanes), dtype=x.dtype)
    for p in range(T):
        pool[p // 64, :, p % 64] = x[p]
    return pool


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,softcap,T,past", [(None, 5.0, 200, 0), (64, None, 200, 0), (65, 3.0, 131, 100), (1, 2.0, 40, 0),
                                                   (7, 30.0, 1, 190), (300, 8.0, 1, 700)])
def test_attention_kernel_caps_scores_and_keeps_the_window(dtype, window, softcap, T, past):
    """``T`` query tokens on top of ``past`` cached keys, against the plain scores, mask and softmax; the single-token
    cases also cut the keys into splits."""
    g = torch.Generator().manual_seed(T + past)
    nq, nkv, d, dv, scale, total = 4, 2, 12, 20, 0.7, past + T
    q = torch.randn(T, nq, d, generator=g).to(dtype)
    k = torch.randn(total, nkv, d, generator=g).to(dtype)
    v = torch.randn(total, nkv, dv, generator=g).to(dtype)
    n_pages = -(-total // 64)
    out = torch.empty((T, nq * dv), dtype=dtype, device="cuda")
    ints = lambda *values: torch.tensor(values, dtype=torch.int32, device="cuda")
    for splits in ((1, 3) if T == 1 else (1,)):
        partial = torch.empty(T * nq * splits * (dv + 2), dtype=torch.float32, device="cuda") if splits > 1 else None
        ops.attention_simt(q.view(T, -1).cuda(), _paged(k, n_pages).cuda(), _paged(v, n_pages).cuda(), out, ints(0, T), ints(past),
                           ints(0, n_pages), torch.arange(n_pages, dtype=torch.int32, device="cuda"), n_seqs=1, max_q_len=T,
                           nq=nq, nkv=nkv, d=d, dv=dv, page_size=64, ring_pages=0, window=window or 0, scale=scale,
                           splits=splits, partial=partial, softcap=softcap or 0.0)
        see = plain.visible(total, window)[past:]
        for head in range(nq):
            s = plain.capped_scores(q[:, head].double(), k[:, head // 2].double(), scale, softcap)
            want = torch.softmax(s.masked_fill(~see, float("-inf")), -1) @ v[:, head // 2].double()
            got = out.view(T, nq, dv)[:, head].cpu().double()
            assert (got - want).abs().max() < (2e-5 if dtype == torch.float32 else 2e-2), (head, splits)


@pytest.mark.parametrize("d,dv", [(32, 48), (16, 16), (80, 32), (128, 128), (64, 64)])
@pytest.mark.parametrize("window,softcap,T,past,ring", [(None, 5.0, 200, 0, 0), (64, None, 200, 0, 0), (65, 3.0, 131, 100, 0),
                                                        (1, 2.0, 40, 0, 0), (7, 30.0, 1, 190, 0), (100, 8.0, 300, 500, 8),
                                                        (129, 20.0, 2, 1000, 5), (70, 9.0, 64, 64, 4), (129, 20.0, 1, 1001, 5), (None, 6.0, 1, 333, 0)])
def test_tensor_core_attention_caps_scores_and_keeps_the_window(d, dv, window, softcap, T, past, ring):
    """The bfloat16 tensor-core form against the plain scores, mask and softmax: prompts, portions on top of cached
    keys, pages and rings of pages (a ring holds the window and the portion, older positions are overwritten)."""
    g = torch.Generator().manual_seed(T + past + d)
    nq, nkv, scale, total = 4, 2, 1.5 / d ** 0.5, past + T
    q = torch.randn(T, nq, d, generator=g).bfloat16()
    k = torch.randn(total, nkv, d, generator=g).bfloat16()
    v = torch.randn(total, nkv, dv, generator=g).bfloat16()
    n_pages = ring or -(-total // 64)
    pools = []
    for x in (k, v):
        pool = torch.zeros((n_pages, nkv, 64, x.shape[-1]), dtype=x.dtype)
        for p in range(max(0, total - n_pages * 64) if ring else 0, total):       # later positions overwrite older ones
            pool[(p // 64) % n_pages, :, p % 64] = x[p]
        pools.append(pool.cuda())
    out = torch.empty((T, nq * dv), dtype=torch.bfloat16, device="cuda")
    ints = lambda *values: torch.tensor(values, dtype=torch.int32, device="cuda")
    ops.attention_capped(q.view(T, -1).cuda(), pools[0], pools[1], out, ints(0, T), ints(past), ints(0, n_pages),
                         torch.arange(n_pages, dtype=torch.int32, device="cuda"), n_seqs=1, max_q_len=T, nq=nq, nkv=nkv, d=d,
                         dv=dv, page_size=64, ring_pages=ring, window=window or 0, scale=scale, softcap=softcap or 0.0)
    see = plain.visible(total, window)[past:]
    want = []
    for head in range(nq):
        s = plain.capped_scores(q[:, head].double(), k[:, head // 2].double(), scale, softcap)
        want.append(torch.softmax(s.masked_fill(~see, float("-inf")), -1) @ v[:, head // 2].double())
        assert (out.view(T, nq, dv)[:, head].cpu().double() - want[-1]).abs().max() < 2e-2, head
    if d == dv and d in ops.TCGEN05_ATTENTION_HEAD_DIMS and T > 16:
        # the kernel that keeps scores and outputs in tensor memory takes the same window, ring and cap
        out.zero_()
        ops.attention_tcgen05(q.view(T, -1).cuda(), pools[0], pools[1], out, ints(0, T), ints(past), ints(0, n_pages),
                              torch.arange(n_pages, dtype=torch.int32, device="cuda"), n_seqs=1, max_q_len=T, nq=nq, nkv=nkv, d=d,
                              page_size=64, scale=scale, window=window or 0, ring_pages=ring, softcap=softcap or 0.0)
        torch.cuda.synchronize()
        ops.raise_on_kernel_fault()
        for head in range(nq):
            assert (out.view(T, nq, dv)[:, head].cpu().double() - want[head]).abs().max() < 2e-2, ("tcgen05", head)
    if T == 1:
        # the form for single tokens, whose blocks take a share of the visible keys each (some shares may be empty)
        for splits in (1, 2, 3, 7):
            out.zero_()
            partial = torch.empty(nq * splits * (dv + 2), dtype=torch.float32, device="cuda") if splits > 1 else None
            ops.attention_capped_decode(q.view(T, -1).cuda(), pools[0], pools[1], out, ints(0, T), ints(past), ints(0, n_pages),
                                        torch.arange(n_pages, dtype=torch.int32, device="cuda"), n_seqs=1, nq=nq, nkv=nkv, d=d,
                                        dv=dv, page_size=64, ring_pages=ring, window=window or 0, scale=scale,
                                        softcap=softcap or 0.0, splits=splits, partial=partial)
            for head in range(nq):
                assert (out.view(T, nq, dv)[:, head].cpu().double() - want[head]).abs().max() < 2e-2, (head, splits)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("where", ["prompt", "decoded"])
def test_one_outstanding_key_shows_both_edges_of_the_window(dtype, where):
    """All keys are alike but one, which matches the query: with the key on the window's last position the output is
    its value, one position further back it is gone.  The same at a page border, and for the newest key."""
    nq = nkv = 1
    d, dv, window, scale = 16, 16, 70, 4.0
    ints = lambda *values: torch.tensor(values, dtype=torch.int32, device="cuda")
    for pos in (69, 127, 128, 200):                       # the query's position
        for back, seen in ((0, True), (window - 1, True), (window, False), (pos, pos < window)):
            if back > pos:
                continue
            total = pos + 1
            k = torch.zeros(total, 1, d)
            k[:, 0, 0] = 1.0                                   # every key: orthogonal to the query
            k[pos - back, 0] = torch.tensor([0.0, 1.0] + [0.0] * (d - 2))
            v = torch.zeros(total, 1, dv)
            v[pos - back, 0, 1] = 1.0
            q_rows = torch.zeros(total, 1, d)
            q_rows[:, 0, 1] = 8.0
            T, past = (total, 0) if where == "prompt" else (1, pos)
            q = q_rows[past:].to(dtype)
            n_pages = -(-total // 64)
            out = torch.empty((T, dv), dtype=dtype, device="cuda")
            common = dict(n_seqs=1, max_q_len=T, nq=nq, nkv=nkv, d=d, dv=dv, page_size=64, ring_pages=0, window=window,
                          scale=scale, softcap=50.0)
            tables = (ints(0, T), ints(past), ints(0, n_pages), torch.arange(n_pages, dtype=torch.int32, device="cuda"))
            ops.attention_simt(q.view(T, -1).cuda(), _paged(k.to(dtype), n_pages).cuda(), _paged(v.to(dtype), n_pages).cuda(), out,
                               *tables, **common)
            weight = float(out[-1, 1])
            assert (weight > 0.99) if seen else (weight == 0.0), (pos, back, weight)
            if dtype == torch.bfloat16:                      # the tensor-core form
                out.zero_()
                ops.attention_capped(q.view(T, -1).cuda(), _paged(k.to(dtype), n_pages).cuda(), _paged(v.to(dtype), n_pages).cuda(),
                                     out, *tables, **common)
                weight = float(out[-1, 1])
                assert (weight > 0.99) if seen else (weight == 0.0), (pos, back, weight)
                if T == 1:
                    for splits in (1, 2):
                        out.zero_()
                        partial = torch.empty(splits * (dv + 2), dtype=torch.float32, device="cuda")
                        decode = {key: value for key, value in common.items() if key != "max_q_len"}
                        ops.attention_capped_decode(q.view(T, -1).cuda(), _paged(k.to(dtype), n_pages).cuda(),
                                                    _paged(v.to(dtype), n_pages).cuda(), out, *tables, splits=splits,
                                                    partial=partial, **decode)
                        weight = float(out[-1, 1])
                        assert (weight > 0.99) if seen else (weight == 0.0), (pos, back, weight, splits)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activation_norm_and_add_gate_and_cap(dtype):
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(9, 50, generator=g) * 2).to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    out = torch.empty_like(x, device="cuda")
    ops.activation(x.cuda(), out, "gelu_erf")
    assert (out.cpu().double() - plain.gelu_erf(x.double())).abs().max() < tol
    ops.activation(x.cuda(), out, "gelu_tanh")
    z = x.double()
    assert (out.cpu().double() - 0.5 * z * (1 + torch.tanh((2 / torch.pi) ** 0.5 * (z + 0.044715 * z ** 3)))).abs().max() < tol
    # the norm after a sublayer and the residual add, in fp32 whatever the compute dtype
    hidden, y, w = torch.randn(9, 50, generator=g), torch.randn(9, 50, generator=g) * 3, torch.randn(50, generator=g)
    h = hidden.clone().cuda()
    ops.rmsnorm_add(h, y.cuda(), w.cuda(), 1e-3)
    assert (h.cpu().double() - (hidden.double() + plain.rms_norm(y.double(), w.double(), 1e-3))).abs().max() < 1e-5
    for width in (50, 48, 2048):                # element by element; four lanes at a time; several per thread
        hid, ys = torch.randn(5, width, generator=g), torch.randn(5, width, generator=g) * 2
        w1, w2 = torch.randn(width, generator=g), torch.randn(width, generator=g)
        h, fused = hid.clone().cuda(), torch.empty((5, width), dtype=dtype, device="cuda")
        want_h = hid.double() + plain.rms_norm(ys.double(), w1.double(), 1e-3)
        if ops.rmsnorm_add_norm(h, ys.cuda(), w1.cuda(), 1e-3, w2.cuda(), 1e-5, fused):
            assert (h.cpu().double() - want_h).abs().max() < 1e-5
            assert (fused.cpu().double() - plain.rms_norm(want_h, w2.double(), 1e-5)).abs().max() < tol * 3
        else:
            assert width % 4 != 0 and torch.equal(h.cpu(), hid)
    # a shared expert's output times sigmoid(sg . x)
    acc, sg = torch.randn(9, 30, generator=g), (torch.randn(50, generator=g) * 0.3).to(dtype)
    for y_dtype in {torch.float32, dtype}:
        ys = torch.randn(9, 30, generator=g).to(y_dtype)
        a = acc.clone().cuda()
        ops.gated_row_add(a, ys.cuda(), x.cuda(), sg.cuda())
        want = acc.double() + torch.sigmoid(x.double() @ sg.double())[:, None] * ys.double()
        assert (a.cpu().double() - want).abs().max() < 1e-5
    logits = torch.randn(4, 33, generator=g) * 20
    capped = logits.clone().cuda()
    ops.softcap(capped, 7.0)
    assert (capped.cpu().double() - 7.0 * torch.tanh(logits.double() / 7.0)).abs().max() < 1e-5
    both = torch.empty((9, 100), dtype=dtype, device="cuda")
    ops.concat_cast(hidden.cuda(), y.cuda(), both)
    assert torch.equal(both.cpu(), torch.cat([hidden, y], -1).to(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,experts,top,K,F", [(1, 5, 2, 40, 24), (6, 3, 1, 44, 12), (700, 7, 3, 48, 16), (90, 1, 1, 24, 8)])
def test_table_routed_experts_against_a_loop_over_tokens(dtype, tokens, experts, top, K, F):
    g = torch.Generator().manual_seed(tokens)
    vocab = 19
    table = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(vocab)]).int()
    ids_in = torch.randint(0, vocab, (tokens,), generator=g).int()
    x = torch.randn(tokens, K, generator=g).to(dtype)
    w_up = (torch.randn(experts, F, K, generator=g) / K ** 0.5).to(dtype)
    w_down = (torch.randn(experts, K, F, generator=g) / F ** 0.5).to(dtype)
    ids = torch.empty((tokens, top), dtype=torch.int32, device="cuda")
    weights = torch.empty((tokens, top), dtype=torch.float32, device="cuda")
    ops.moe_table_route(table.cuda(), ids_in.cuda(), ids, weights, n_experts=experts, weight=1.0 / top)
    assert torch.equal(ids.cpu(), table[ids_in.long()]) and float((weights - 1.0 / top).abs().max()) == 0
    routing = ops.RoutingTable(tokens, top, experts, "cuda", few_rows_ok=ops.grouped_few_rows_ok((K, F), dtype))
    counts = torch.zeros(experts, dtype=torch.int32, device="cuda")
    ops.moe_group(ids, counts, routing)
    act = torch.empty((tokens * top, F), dtype=dtype, device="cuda")
    ops.grouped_gemm_routed(x.cuda(), w_up.cuda(), act, routing, gather=True, epi=ops.GROUPED_GELU_ERF)
    out = torch.empty((tokens * top, K), dtype=torch.float32, device="cuda")
    ops.grouped_gemm_routed(act, w_down.cuda(), out, routing, gather=False, epi=ops.GROUPED_STORE_F32)
    acc = torch.zeros((tokens, K), dtype=torch.float32, device="cuda")
    ops.moe_combine(acc, out, x.cuda(), ids, weights, routing)
    tensors = {"m.table": table}
    for e in range(experts):
        tensors[f"m.e{e}.up"], tensors[f"m.e{e}.down"] = w_up[e].double(), w_down[e].double()
    want = plain.table_experts(x.double(), ids_in.long(), tensors, "m.", {"router": {"top": top}})
    assert (acc.cpu().double() - want).abs().max() < (2e-5 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("tokens,experts,top,K,F", [(7, 5, 3, 616, 1016),       # three chunks of k, the last one partial
                                                    (6, 12, 2, 264, 4096),       # a list long enough for items of 8 weight rows
                                                    (3, 4, 4, 136, 12800),       # the widest rows the form takes
                                                    (1, 2, 1, 8, 8)])
def test_single_token_expert_products_that_walk_item_lists(tokens, experts, top, K, F):
    """bf16 products of a few rows per expert: every warp walks its own list of (tile, weight rows) items."""
    g = torch.Generator().manual_seed(K)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(tokens)]).int().cuda()
    x = torch.randn(tokens, K, generator=g).bfloat16().cuda()
    w_up = (torch.randn(experts, F, K, generator=g) / K ** 0.5).bfloat16().cuda()
    w_down = (torch.randn(experts, K, F, generator=g) / F ** 0.5).bfloat16().cuda()
    assert ops.grouped_few_rows_ok((K, F), torch.bfloat16)
    routing = ops.RoutingTable(tokens, top, experts, "cuda", few_rows_ok=True)
    counts = torch.zeros(experts, dtype=torch.int32, device="cuda")
    ops.moe_group(ids, counts, routing)
    act = torch.empty((tokens * top, F), dtype=torch.bfloat16, device="cuda")
    ops.grouped_gemm_routed(x, w_up, act, routing, gather=True, epi=ops.GROUPED_GELU_ERF)
    out = torch.empty((tokens * top, K), dtype=torch.float32, device="cuda")
    ops.grouped_gemm_routed(act, w_down, out, routing, gather=False, epi=ops.GROUPED_STORE_F32)
    perm = routing.perm[:tokens * top].long()          # sorted row i is pair perm[i] = token * top + choice
    for i in range(tokens * top):
        t, e = int(perm[i]) // top, int(ids.flatten()[perm[i]])
        want = plain.gelu_erf(x[t].double() @ w_up[e].double().T)
        assert ((act[i].double() - want).abs() <= 2e-2 + 1e-2 * want.abs()).all()
        want = act[i].double() @ w_down[e].double().T
        assert (out[i].double() - want).abs().max() < 1e-4


# ----------------------------------------------------------------------------- whole models


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["A", "B", "C", "bare", "wide"])
def test_whole_prompts_and_their_first_tokens(case, dtype, tmp_path_factory):
    model = engine(case, dtype, tmp_path_factory)
    cfg = CONFIGS[case][0]
    cache = model.make_cache(max_tokens=512, max_seqs=2)
    for n in (1, 2, 3, 150):
        tokens = plain.random_prompts(cfg, [n], n)[0]
        slot = cache.alloc()
        got = model.step(cache, [slot], [tokens], "all")
        cache.free(slot)
        if n >= 10 or dtype == "float32":
            close(got, expected(case, tokens), dtype, f"{case} whole prompt of {n}")
    cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_residual_stream_after_every_layer_run(dtype, tmp_path_factory):
    """The stream after each execution (looped layers count each time) against the plain implementation's."""
    model = engine("A", dtype, tmp_path_factory)
    tokens = plain.random_prompts(plain.TINY_A, [40], 2)[0]
    want = plain.forward(plain.TINY_A, weights_of("A"), tokens)[1].float()
    seen, blocks = [], [layer for layer in model.decoder.layers if type(layer).__name__ == "SandwichBlock"]
    originals = [block.forward for block in blocks]
    try:
        for block, original in zip(blocks, originals):
            def record(hidden, ctx, view, original=original):
                result = original(hidden, ctx, view)
                flush_residual_add(ctx)           # the block leaves its last add to the next norm
                seen.append(hidden.clone())
                return result
            block.forward = record
        cache = model.make_cache(max_tokens=64, max_seqs=1)
        model.step(cache, [cache.alloc()], [tokens], "last")
    finally:
        for block, original in zip(blocks, originals):
            block.forward = original
    assert len(seen) == want.shape[0] == 8
    for run, (got, ref) in enumerate(zip(seen, want)):
        bound = 1e-4 if dtype == "float32" else 0.03 * float(ref.abs().max())
        assert float((got.cpu() - ref).abs().max()) < bound, run


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["A", "B", "C", "wide"])
def test_prompt_then_single_tokens_over_page_and_window_borders(case, dtype, tmp_path_factory):
    model = engine(case, dtype, tmp_path_factory)
    cfg = CONFIGS[case][0]
    tokens = plain.random_prompts(cfg, [150], 4)[0]
    want = expected(case, tokens)
    cache = model.make_cache(max_tokens=192, max_seqs=1)
    slot = cache.alloc()
    rows = [model.step(cache, [slot], [tokens[:50]], "all")]
    rows += [model.step(cache, [slot], [[t]], "last") for t in tokens[50:]]         # past 64, 70, 128, 130
    close(torch.cat(rows), want, dtype, f"{case} decoded")
    cache.free(slot)
    slot = cache.alloc()                                                            # the same slot and pages again
    rows = [model.step(cache, [slot], [[t]], "last") for t in tokens[:80]]          # from the very first token
    close(torch.cat(rows), want[:80], dtype, f"{case} decoded from the first token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["A", "C", "wide"])
def test_portions_of_several_sizes_down_to_two_tokens(case, dtype, tmp_path_factory):
    model = engine(case, dtype, tmp_path_factory)
    cfg = CONFIGS[case][0]
    tokens = plain.random_prompts(cfg, [200], 5)[0]
    want = expected(case, tokens)
    for sizes in ([2] * 40 + [120], [63, 2, 64, 1, 70], [7, 129, 64], [199, 1]):
        cache = model.make_cache(max_tokens=256, max_seqs=1)
        slot, at, rows = cache.alloc(), 0, []
        for size in sizes:
            rows.append(model.step(cache, [slot], [tokens[at:at + size]], "all"))
            at += size
        close(torch.cat(rows), want, dtype, f"{case} portions {sizes[:4]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ["A", "B", "wide"])
def test_unequal_batches_on_slots_and_pages_used_again(case, dtype, tmp_path_factory):
    model = engine(case, dtype, tmp_path_factory)
    cfg = CONFIGS[case][0]
    requests = plain.random_prompts(cfg, [90, 1, 33, 70, 5, 129], 8)
    cache = model.make_cache(max_tokens=448, max_seqs=3)
    got = {r: [] for r in range(len(requests))}
    for batch in ([0, 1, 2], [3, 4, 5]):          # the second batch takes the slots and pages the first gave back
        slots = {r: cache.alloc() for r in batch}
        cut = {r: max(1, len(requests[r]) - 4 - 2 * (r % 3)) for r in batch}
        logits = model.step(cache, [slots[r] for r in batch], [requests[r][:cut[r]] for r in batch], "all")
        at = 0
        for r in batch:
            got[r].append(logits[at:at + cut[r]])
            at += cut[r]
        live = list(batch)
        while live:
            for r in [r for r in live if cut[r] == len(requests[r])]:
                cache.free(slots.pop(r))
                live.remove(r)
            if not live:
                break
            logits = model.step(cache, [slots[r] for r in live], [[requests[r][cut[r]]] for r in live], "last")
            for i, r in enumerate(live):
                got[r].append(logits[i:i + 1])
                cut[r] += 1
        cache.check()
    for r, tokens in enumerate(requests):
        if dtype == "float32":
            close(torch.cat(got[r]), expected(case, tokens), dtype, f"{case} batched request {r}")
    close(torch.cat([row for r in range(len(requests)) for row in got[r]]),
          torch.cat([expected(case, tokens) for tokens in requests]), dtype, f"{case} batched requests")


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_rows_do_not_depend_on_their_neighbours(dtype, tmp_path_factory):
    model = engine("A", dtype, tmp_path_factory)
    requests = plain.random_prompts(plain.TINY_A, [77, 12, 140], 6)
    cache = model.make_cache(max_tokens=512, max_seqs=4)
    alone = []
    for tokens in requests:
        slot = cache.alloc()
        alone.append(model.step(cache, [slot], [tokens], "all"))
        cache.free(slot)
    slots = [cache.alloc() for _ in requests]
    together = model.step(cache, slots, requests, "all")
    gap = (together - torch.cat(alone)).abs().max()
    assert float(gap) < (1e-5 if dtype == "float32" else 5e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sharp_attention_finds_far_keys_in_prompts_and_in_decoding(dtype, tmp_path_factory):
    """Scores of up to 24 make the softmax pick single keys anywhere in a window of 300 positions: a key that is
    lost, read from the wrong page or dropped one position early moves the logits.  float32 is held to the plain
    implementation; bfloat16 (whose rounded scores such a scale magnifies) to its own whole-prompt run, which the
    decoded run must repeat from the cache."""
    model = engine("sharp", dtype, tmp_path_factory)
    tokens = plain.random_prompts(plain.SHARP, [700], 9)[0]
    cache = model.make_cache(max_tokens=1536, max_seqs=2)
    whole = cache.alloc()
    whole_logits = model.step(cache, [whole], [tokens], "all")
    want = expected("sharp", tokens) if dtype == "float32" else whole_logits
    if dtype == "float32":
        close(whole_logits, want, dtype, "sharp whole")
    decoded = cache.alloc()
    rows = [model.step(cache, [decoded], [tokens[:500]], "all")]
    rows += [model.step(cache, [decoded], [[t]], "last") for t in tokens[500:]]
    close(torch.cat(rows), want, dtype, "sharp decoded")
    if dtype == "float32":
        # the plain logits really depend on keys hundreds of positions back, and on the window's exact size
        near_only = plain.forward(plain.SHARP, weights_of("sharp"), tokens[500:])[0].float()
        assert float((near_only[-20:] - want[-20:]).abs().max()) > 0.05
        import copy
        narrower = copy.deepcopy(plain.SHARP)
        narrower["layers"][0]["mixer"]["mask"]["size"] = 299
        off_by_one = plain.forward(narrower, weights_of("sharp"), tokens)[0].float()
        assert float((off_by_one[300:] - want[300:]).abs().max()) > 0.05


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_prompts_are_cut_and_go_round_the_ring(dtype, tmp_path_factory):
    """A prompt of 700 tokens on a cache whose passes take 256 tokens of a sequence: three portions, the third one
    written over the ring's oldest pages (window 100: seven pages), beside a short request in the same step; heads
    of 64 lanes, so bfloat16 takes the kernel that keeps scores in tensor memory."""
    model = engine("wide", dtype, tmp_path_factory)
    long, short = plain.random_prompts(plain.WIDE_HEADS, [700, 40], 12)
    cache = model.make_cache(max_tokens=1024, max_seqs=2)
    assert cache.max_step_tokens == 256 and any(0 < group.ring_pages * 64 < 700 for group in cache.kv_groups)
    slots = [cache.alloc(), cache.alloc()]
    got = model.step(cache, slots, [long, short], "all")
    close(got[:700], expected("wide", long), dtype, "long prompt in portions")
    close(got[700:], expected("wide", short), dtype, "short prompt beside it")
    more = plain.random_prompts(plain.WIDE_HEADS, [30], 13)[0]
    rows = [model.step(cache, slots[:1], [[t]], "last") for t in more]
    close(torch.cat(rows), expected("wide", long + more)[700:], dtype, "single tokens after the long prompt")


def test_long_decoding_wraps_the_ring_of_a_windowed_cache(tmp_path_factory):
    """Windows of 7 and 3 keep rings of a few pages per sequence; 700 single-token steps go round them twice."""
    model = engine("A", "float32", tmp_path_factory)
    tokens = plain.random_prompts(plain.TINY_A, [720], 11)[0]
    want = expected("A", tokens)
    cache = model.make_cache(max_tokens=768, max_seqs=1)
    slot = cache.alloc()
    rows = [model.step(cache, [slot], [tokens[:20]], "all")]
    rows += [model.step(cache, [slot], [[t]], "last") for t in tokens[20:]]
    close(torch.cat(rows), want, "float32", "long decoding")
    assert any(group.ring_pages and 720 > group.ring_pages * 64 for group in cache.kv_groups)


def test_decode_steps_are_captured_as_graphs(tmp_path_factory):
    assert engine("A", "bfloat16", tmp_path_factory).decoder.graph_safe


def test_greedy_generation_through_the_entry_point(tmp_path_factory):
    for case in ("A", "B"):
        model = engine(case, "float32", tmp_path_factory)
        cfg = CONFIGS[case][0]
        prompts = plain.random_prompts(cfg, [9, 30, 3], 10)
        weights = weights_of(case)
        for use_graphs in (False, True):              # the step function, then the captured decode steps
            result = model.generate(prompts, max_new_tokens=6, use_graphs=use_graphs)
            for prompt, produced in zip(prompts, result.generated_ids):
                assert len(produced) == 6
                ids = list(prompt)
                for token in produced:
                    logits = plain.forward(cfg, weights, ids)[0][-1]
                    assert float(logits.max() - logits[token]) < 1e-4, "the generated token is not the plain argmax"
                    ids.append(token)


def test_command_line_writes_a_random_model_and_generates_from_it(tmp_path):
    cfg = plain.TINY_B
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    root = Path(__file__).resolve().parent.parent
    run = lambda *a: subprocess.run([sys.executable, "-m", "ondeviceinfer_b200", *a], cwd=root, text=True,
                                    capture_output=True, timeout=600)
    made = run("random-model", "--config", str(tmp_path / "config.json"), "--seed", "3", "--out", str(tmp_path / "model"))
    assert made.returncode == 0, made.stderr
    done = run("generate", "--model", str(tmp_path / "model"), "--prompt-ids", "5,9,2,40,7", "--dtype", "float32",
               "--max-new-tokens", "4", "--warmup-runs", "0", "--repeats", "1", "--output", str(tmp_path / "report.json"))
    assert done.returncode == 0, done.stderr
    report = json.loads((tmp_path / "report.json").read_text())
    from ondeviceinfer_b200.weights import SafetensorsSource
    source = SafetensorsSource(tmp_path / "model")
    weights = {n: source.fetch(n) for n in source.stored()}
    ids = [5, 9, 2, 40, 7]
    for token in report["measurements"][0]["output_token_ids"]:
        logits = plain.forward(cfg, weights, ids)[0][-1]
        assert float(logits.max() - logits[token]) < 1e-4
        ids.append(token)
    assert len(ids) == 9


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("seed", range(8))
def test_models_of_random_odd_sizes(seed, dtype, tmp_path):
    """Configurations drawn from odd sizes: a prompt, then single tokens, then a portion, on a cache that a shorter
    request used before."""
    cfg = plain.random_config(seed)
    weights = plain.random_weights(cfg, 300 + seed)
    model = odi.load_resident_model(write_model_folder(tmp_path / "model", cfg, weights), dtype=dtype)
    tokens = plain.random_prompts(cfg, [150], seed)[0]
    want = plain.forward(cfg, weights, tokens)[0].float()
    cache = model.make_cache(max_tokens=192, max_seqs=1)
    slot = cache.alloc()
    model.step(cache, [slot], [tokens[:37]], "none")
    cache.free(slot)
    slot = cache.alloc()
    rows = [model.step(cache, [slot], [tokens[:100]], "all")]
    rows += [model.step(cache, [slot], [[t]], "last") for t in tokens[100:130]]
    rows.append(model.step(cache, [slot], [tokens[130:]], "all"))
    close(torch.cat(rows), want, dtype, f"random sizes {seed}: {json.dumps(cfg)[:300]}")
