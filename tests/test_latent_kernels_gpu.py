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
@pytest.mark.parametrize("T,E,top,width,ff", [(1, 4, 2, 32, 16), (5, 3, 3, 40, 24), (300, 16, 4, 64, 96), (130, 7, 1, 36, 20), (64, 64, 8, 128, 64)])
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
