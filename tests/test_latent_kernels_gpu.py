"""The kernels behind attention over a latent and routed experts, each alone against plain float32 PyTorch: products
with one matrix per head or per expert (the tensor-core tiles, and the FFMA tiles that odd sizes and float32 take),
routing, grouping, the weighted sum over a token's experts, a factor per channel."""
import pytest
import torch

from sandyrt_b200.csrc import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _rand(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (scale * torch.randn(*shape, generator=g)).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("T,G,N,K,a_gcols,o_gcols", [
    (1, 3, 24, 16, 24, 32),          # one token; heads wider than what the product reads and writes
    (70, 5, 40, 64, 64, 40),         # dense heads, more than one row tile
    (9, 2, 100, 36, 40, 104),        # sizes that divide by nothing: K no multiple of 8 (FFMA tiles in both types)
    (200, 4, 64, 128, 128, 64),      # the sizes of a real layer
    (33, 1, 8, 8, 8, 8),
])
def test_head_product(T, G, N, K, a_gcols, o_gcols, dtype, tol):
    a = _rand(T, G * a_gcols, dtype=dtype, seed=1)
    w = _rand(G * N, K, dtype=dtype, seed=2, scale=K ** -0.5)
    out = torch.full((T, G * o_gcols), 7.0, dtype=dtype, device=DEV)
    ops.head_product(a, w, out, n_groups=G, a_gcols=a_gcols, o_gcols=o_gcols)
    af, wf = a.float().view(T, G, a_gcols)[:, :, :K], w.float().view(G, N, K)
    want = torch.einsum("tgk,gnk->tgn", af, wf)
    got = out.float().view(T, G, o_gcols)
    assert torch.allclose(got[:, :, :N], want, atol=tol, rtol=tol)
    assert torch.all(got[:, :, N:] == 7.0)                     # nothing written beside a head's own columns


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 1.5e-2)])
@pytest.mark.parametrize("T,E,top,width,ff", [(1, 4, 2, 32, 16), (5, 3, 3, 40, 24), (300, 16, 4, 64, 96), (130, 7, 1, 36, 20), (64, 64, 8, 128, 64), (20, 48, 40, 32, 16)])
def test_routed_experts_from_logits_to_sum(T, E, top, width, ff, dtype, tol):
    h = _rand(T, width, dtype=dtype, seed=3)
    logits = _rand(T, E, seed=4, scale=2.0)
    bias = _rand(E, seed=5)
    up = _rand(E * ff, width, dtype=dtype, seed=6, scale=width ** -0.5)
    down = _rand(E * width, ff, dtype=dtype, seed=7, scale=ff ** -0.5)
    r = ops.moe_route(logits, bias, top)
    z = logits + bias
    want_idx = z.topk(top, -1).indices                                      # descending, as the kernel chooses
    assert torch.equal(r.expert_of.view(T, top).long(), want_idx)
    want_w = torch.softmax(z.gather(1, want_idx), -1)
    assert torch.allclose(r.weight_of.view(T, top), want_w, atol=1e-6)
    # grouping: a permutation whose slots are sorted by expert
    start, slot_of, entry_of = r.group_start.cpu(), r.slot_of_entry.cpu().long(), r.entry_of_slot.cpu().long()
    assert start[0] == 0 and start[-1] == T * top and torch.equal(entry_of[slot_of], torch.arange(T * top))
    experts = r.expert_of.cpu().long()
    for e in range(E):
        assert torch.all(experts[entry_of[start[e]:start[e + 1]]] == e)
    inner = torch.empty(T * top, ff, dtype=dtype, device=DEV)
    ops.expert_product(r, h, up, inner, gather=True, act="relu_squared")
    rows = torch.empty(T * top, width, dtype=torch.float32, device=DEV)
    ops.expert_product(r, inner, down, rows, gather=False)
    y = torch.full((T, width), 0.5, device=DEV)
    ops.moe_combine(r, rows, y, add=True)
    want = torch.full((T, width), 0.5, device=DEV)
    upf, downf = up.float().view(E, ff, width), down.float().view(E, width, ff)
    for j in range(top):
        e = want_idx[:, j]
        a = torch.relu(torch.einsum("tk,tnk->tn", h.float(), upf[e])) ** 2
        if dtype == torch.bfloat16:
            a = a.to(dtype).float()
        want += want_w[:, j:j + 1] * torch.einsum("tk,tnk->tn", a, downf[e])
    assert torch.allclose(y, want, atol=tol * 4, rtol=tol)
    y2 = torch.empty_like(y)
    ops.moe_combine(r, rows, y2, add=False)
    assert torch.allclose(y2, y - 0.5, atol=1e-5)


@pytest.mark.parametrize("T,E,top,width,ff", [(300, 16, 4, 64, 96), (1, 4, 2, 32, 16), (700, 5, 2, 200, 136), (1500, 3, 1, 72, 40)])
def test_expert_products_on_tcgen05(T, E, top, width, ff):
    """The same two products through the tcgen05 kernel (rows gathered into the slots' order first), against float32
    PyTorch and against the mma.sync tiles: groups that start anywhere, tiles cut by a group's end and by N."""
    dtype = torch.bfloat16
    h = _rand(T, width, dtype=dtype, seed=3)
    r = ops.moe_route(_rand(T, E, seed=4, scale=2.0), None, top)
    up = _rand(E * ff, width, dtype=dtype, seed=6, scale=width ** -0.5)
    down = _rand(E * width, ff, dtype=dtype, seed=7, scale=ff ** -0.5)
    sorted_rows = torch.empty(T * top, width, dtype=dtype, device=DEV)
    ops.moe_gather(r, h, sorted_rows)
    token_of_slot = (r.entry_of_slot.long() // top)
    assert torch.equal(sorted_rows, h[token_of_slot])
    inner = torch.full((T * top, ff), 3.0, dtype=dtype, device=DEV)
    ops.expert_product_tc(r, sorted_rows, up, inner, act="relu_squared")
    inner_mma = torch.empty_like(inner)
    ops.expert_product(r, h, up, inner_mma, gather=True, act="relu_squared")
    expert_of_slot = r.expert_of.long()[r.entry_of_slot.long()]
    want = torch.relu(torch.einsum("sk,snk->sn", sorted_rows.float(), up.float().view(E, ff, width)[expert_of_slot])) ** 2
    assert torch.allclose(inner.float(), want, atol=2e-2, rtol=2e-2)
    assert torch.allclose(inner.float(), inner_mma.float(), atol=2e-2, rtol=2e-2)
    rows = torch.full((T * top, width), 3.0, dtype=torch.float32, device=DEV)
    ops.expert_product_tc(r, inner, down, rows)
    want = torch.einsum("sk,snk->sn", inner.float(), down.float().view(E, width, ff)[expert_of_slot])
    assert torch.allclose(rows, want, atol=2e-2, rtol=2e-2)
    ops.check_kernel_status(rows.device)


def test_equal_logits_go_to_the_lower_expert():
    logits = torch.zeros(3, 6, device=DEV)
    logits[1, 4] = logits[1, 2] = 1.0
    r = ops.moe_route(logits, None, 3)
    assert r.expert_of.view(3, 3).tolist() == [[0, 1, 2], [2, 4, 0], [0, 1, 2]]


def test_channel_scale_joins_one_or_two_branches():
    x, y1, y2 = _rand(37, 50, seed=1), _rand(37, 50, seed=2), _rand(37, 50, seed=3)
    g1, g2 = _rand(50, seed=4), _rand(50, seed=5)
    want = x + g1 * y1
    ops.scale_add(y1, g1, x)
    assert torch.allclose(x, want, atol=1e-6)
    want = x + (g1 * y1 + g2 * y2)
    ops.scale_add(y1, g1, x, y2, g2)
    assert torch.allclose(x, want, atol=1e-6)


# ---- single-token attention with the heads of a group as the rows of one product ----------------------------------
def _paged(keys, values, page_size, n_kv_heads, seed):
    """Scatter per-request keys/values [len, Hkv, D] into a poisoned paged cache with shuffled pages; one plane when
    `values` is None.  Returns the views, the block table and the lengths."""
    lens = [k.shape[0] for k in keys]
    D = keys[0].shape[2]
    blocks = [-(-n // page_size) for n in lens]
    n_pages = sum(blocks) + 3
    planes = 1 if values is None else 2
    arena = torch.full((n_pages, planes, n_kv_heads, page_size, D), float("nan"), dtype=torch.bfloat16, device=DEV)
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    table = torch.full((len(keys), max(blocks)), -1, dtype=torch.int32)
    for r, k in enumerate(keys):
        for b in range(blocks[r]):
            page = order.pop()
            table[r, b] = page
            n = min(page_size, lens[r] - b * page_size)
            arena[page, 0, :, :n] = k[b * page_size:b * page_size + n].transpose(0, 1)
            arena[page, 0, :, n:] = float("nan")
            if values is not None:
                arena[page, 1, :, :n] = values[r][b * page_size:b * page_size + n].transpose(0, 1)
    k_view = arena[:, 0]
    v_view = arena[:, 1] if values is not None else k_view
    return k_view, v_view, table.to(DEV), lens


@pytest.mark.parametrize("H,Hkv,D,page_size,splits,one_plane", [
    (12, 1, 128, 16, 1, True), (12, 1, 128, 16, 5, True), (24, 1, 80, 16, 3, True), (5, 1, 16, 8, 2, True),
    (8, 2, 64, 16, 4, False), (40, 2, 48, 32, 7, False), (16, 1, 112, 16, 64, True),
])
def test_decode_attention_with_heads_as_rows(H, Hkv, D, page_size, splits, one_plane):
    g = torch.Generator().manual_seed(H * 1000 + D)
    lens = [1, 17, 300, 64, 129]
    keys = [torch.randn(n, Hkv, D, generator=g).to(torch.bfloat16).to(DEV) for n in lens]
    values = None if one_plane else [torch.randn(n, Hkv, D, generator=g).to(torch.bfloat16).to(DEV) for n in lens]
    k_view, v_view, table, _ = _paged(keys, values, page_size, Hkv, seed=D)
    T = len(lens)
    q = (2.0 * torch.randn(T, H * D, generator=g)).to(torch.bfloat16).to(DEV)
    q[2] *= 3.0                                                   # sharp scores on the long request: single far keys win
    sink = torch.randn(H, generator=g).to(DEV)
    gate = torch.rand(T, H, generator=g).to(DEV)
    token_seq = torch.arange(T, dtype=torch.int32, device=DEV)
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    scale = D ** -0.5
    for use_sink, use_gate in ((False, False), (True, True)):
        out = torch.full((T, H * D), 9.0, dtype=torch.bfloat16, device=DEV)
        ops.decode_attention_shared(q, k_view, v_view, table, token_seq, positions, out, n_heads=H, scale=scale, splits=splits,
                                    sink=sink if use_sink else None, out_gate=gate if use_gate else None)
        ops.check_kernel_status(out.device)
        for t in range(T):
            kf = keys[t].float()
            vf = kf if one_plane else values[t].float()
            for h in range(H):
                kv = h // (H // Hkv)
                s = (kf[:, kv] @ q[t, h * D:(h + 1) * D].float()) * scale
                if use_sink:
                    p = torch.softmax(torch.cat([s, sink[h:h + 1]]), 0)[:-1]
                else:
                    p = torch.softmax(s, 0)
                want = p @ vf[:, kv]
                if use_gate:
                    want = want * gate[t, h]
                got = out[t, h * D:(h + 1) * D].float()
                assert torch.allclose(got, want, atol=3e-2, rtol=3e-2), (t, h, float((got - want).abs().max()))
