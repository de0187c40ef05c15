"""Kernels that the hybrid mixers add, each against a plain float64 formula: the sink and the per-head output gate
in every attention kernel, the RMS norm family, the gated activation."""
import math

import pytest
import torch

from test_kernels_gpu import ATT_TOL, DEV, _paged_case

pytestmark = pytest.mark.gpu


def _want(case, H, Hkv, scale, sink, gate, window=0):
    """Softmax attention whose denominator also holds exp(sink[h]); head h's output of token t times gate[t, h]."""
    outs, t = [], 0
    for s, (before, n) in enumerate(case["seqs"]):
        k, v, q = case["dense_k"][s].double(), case["dense_v"][s].double(), case["qs"][s].double()
        for i in range(n):
            pos = before + i
            lo = max(0, pos + 1 - window) if window else 0
            row = []
            for h in range(H):
                kh = h // (H // Hkv)
                sc = (k[lo:pos + 1, kh] @ q[i, h]) * scale
                m = torch.maximum(sc.max(), sink[h])
                p = torch.exp(sc - m)
                row.append((p @ v[lo:pos + 1, kh]) / (p.sum() + torch.exp(sink[h] - m)) * gate[t, h])
            outs.append(torch.cat(row))
            t += 1
    return torch.stack(outs)


def _extras(T, H, seed):
    g = torch.Generator().manual_seed(seed)
    sink = (torch.randn(H, generator=g) * 2.0).double()
    gate = torch.rand(T, H, generator=g).double() + 0.25
    return sink, gate, sink.float().to(DEV), gate.float().to(DEV).contiguous()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv,D,page_size", [(4, 2, 16, 16), (5, 5, 48, 8), (6, 2, 64, 16), (4, 1, 128, 32), (3, 1, 80, 4)])
def test_general_kernel_with_sink_and_gate(dtype, H, Hkv, D, page_size):
    from sandyrt_b200.csrc import ops

    seqs = [(0, 33), (40, 1), (17, 24), (0, 1), (100, 1)]
    case = _paged_case(dtype, H, Hkv, D, page_size, seqs, seed=D + H)
    T = case["q"].shape[0]
    sink, gate, sink_d, gate_d = _extras(T, H, seed=D)
    scale = 0.7 / math.sqrt(D)
    out = torch.full_like(case["q"], float("nan"))
    ops.paged_attention(case["q"], case["kc"], case["vc"], case["table"], case["tok_seq"], case["tok_pos"], out,
                        n_heads=H, scale=scale, sink=sink_d, out_gate=gate_d)
    ops.check_kernel_status(DEV)
    assert (out.double().cpu() - _want(case, H, Hkv, scale, sink, gate)).abs().max().item() < ATT_TOL[dtype] * 1.5
    # a sink far below every score and a gate of one: the plain softmax
    plain_out, off = torch.empty_like(out), torch.empty_like(out)
    ops.paged_attention(case["q"], case["kc"], case["vc"], case["table"], case["tok_seq"], case["tok_pos"], plain_out, n_heads=H, scale=scale)
    ops.paged_attention(case["q"], case["kc"], case["vc"], case["table"], case["tok_seq"], case["tok_pos"], off, n_heads=H, scale=scale,
                        sink=torch.full((H,), -1e4, device=DEV), out_gate=torch.ones(T, H, device=DEV))
    assert torch.equal(off, plain_out)


@pytest.mark.parametrize("kind,dtype,H,Hkv,D,page_size,splits", [
    ("scratch", torch.float32, 4, 2, 32, 16, 1), ("scratch", torch.bfloat16, 3, 3, 64, 16, 5), ("scratch", torch.float32, 2, 1, 128, 32, 3),
    ("cluster", torch.float32, 4, 4, 16, 16, 2), ("cluster", torch.bfloat16, 6, 2, 64, 8, 5), ("cluster", torch.bfloat16, 4, 1, 128, 32, 8),
    ("bulk", torch.bfloat16, 12, 12, 64, 16, 1), ("bulk", torch.float32, 3, 1, 32, 4, 3), ("bulk", torch.bfloat16, 4, 1, 128, 32, 8),
    ("mma", torch.bfloat16, 12, 12, 64, 16, 1), ("mma", torch.bfloat16, 6, 2, 64, 8, 3), ("mma", torch.bfloat16, 5, 5, 64, 16, 8),
])
def test_decode_kernels_with_sink_and_gate(kind, dtype, H, Hkv, D, page_size, splits):
    """Single tokens over 1 to 700 keys through each decode kernel; the sink counts once however many blocks
    share a row's keys."""
    from sandyrt_b200.csrc import ops

    seqs = [(699, 1), (0, 1), (63, 1), (64, 1), (300, 1), (15, 1), (128, 1)]
    case = _paged_case(dtype, H, Hkv, D, page_size, seqs, seed=D + splits)
    T = case["q"].shape[0]
    sink, gate, sink_d, gate_d = _extras(T, H, seed=splits)
    scale = 1.0 / math.sqrt(D)
    out = torch.full_like(case["q"], float("nan"))
    kw = dict(n_heads=H, scale=scale, num_splits=splits, sink=sink_d, out_gate=gate_d)
    if kind == "scratch":
        kw["scratch"] = torch.full((T * H * splits * (D + 2),), float("nan"), dtype=torch.float32, device=DEV)
    else:
        kw[kind] = True
    ops.decode_attention(case["q"], case["kc"], case["vc"], case["table"], case["tok_seq"], case["tok_pos"], out, **kw)
    ops.check_kernel_status(DEV)
    assert (out.double().cpu() - _want(case, H, Hkv, scale, sink, gate)).abs().max().item() < ATT_TOL[dtype] * 1.5


@pytest.mark.parametrize("H,Hkv,D,page_size,tc", [(4, 2, 64, 16, True), (12, 12, 64, 16, True), (4, 2, 64, 16, False), (3, 1, 48, 8, False),
                                                   (2, 2, 128, 32, False), (5, 5, 16, 16, False)])
def test_prompt_kernels_with_sink_and_gate(H, Hkv, D, page_size, tc):
    """Portions of prompts (some behind cached tokens, one longer than a query tile) beside single tokens."""
    from sandyrt_b200.csrc import ops

    seqs = [(0, 150), (40, 1), (17, 70), (0, 1), (200, 3)]
    case = _paged_case(torch.bfloat16, H, Hkv, D, page_size, seqs, seed=D + H, runs=(0,))
    T = case["q"].shape[0]
    sink, gate, sink_d, gate_d = _extras(T, H, seed=H)
    scale = 1.0 / math.sqrt(D)
    q_start = torch.tensor([0] + list(torch.tensor([n for _, n in seqs]).cumsum(0)), dtype=torch.int32, device=DEV)
    kv_before = torch.tensor([b for b, _ in seqs], dtype=torch.int32, device=DEV)
    out = torch.full_like(case["q"], float("nan"))
    ops.prefill_attention(case["q"], case["kc"], case["vc"], case["table"], q_start, kv_before, out, n_heads=H,
                          max_q_len=max(n for _, n in seqs), scale=scale, tc=tc, sink=sink_d, out_gate=gate_d)
    ops.check_kernel_status(DEV)
    assert (out.double().cpu() - _want(case, H, Hkv, scale, sink, gate)).abs().max().item() < ATT_TOL[torch.bfloat16] * 1.5


@pytest.mark.parametrize("width", [48, 100, 256, 777, 1600, 5000])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_and_its_residual_form(width, out_dtype):
    from sandyrt_b200.csrc import ops

    g = torch.Generator().manual_seed(width)
    x = (torch.randn(37, width, generator=g) * 3).to(DEV)
    gain = (1 + 0.3 * torch.randn(width, generator=g)).to(DEV)
    eps = 1e-5
    want = x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + eps) * gain.double()
    rows = torch.tensor([5, 0, 36, 5], dtype=torch.int32, device=DEV)
    out = torch.full((4, width), float("nan"), dtype=out_dtype, device=DEV)
    ops.rmsnorm(x, gain, eps, out, rows=rows)
    tol = 2e-5 if out_dtype == torch.float32 else 3e-2
    assert (out.double() - want[rows.long()]).abs().max().item() < tol
    if out_dtype == torch.float32:
        stream = torch.randn(37, width, generator=g).to(DEV)
        want2 = stream.double() + 0.3 * want
        ops.rmsnorm_add(x, gain, eps, 0.3, stream)
        assert (stream.double() - want2).abs().max().item() < 2e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dim,shared,act", [(4, 32, True, "silu"), (3, 20, False, "sigmoid"), (1, 128, False, "sigmoid"), (2, 200, True, "silu")])
def test_head_norm_with_output_gate(dtype, H, dim, shared, act):
    from sandyrt_b200.csrc import ops

    g = torch.Generator().manual_seed(dim)
    o = (torch.randn(19, H * dim, generator=g) * 2).to(DEV)
    gate = torch.randn(19, H * dim, generator=g).to(dtype).to(DEV)
    gain = (1 + 0.3 * torch.randn(dim if shared else H * dim, generator=g)).to(DEV)
    out = torch.full((19, H * dim), float("nan"), dtype=dtype, device=DEV)
    ops.head_norm_gate(o, gain, gate, out, n_heads=H, eps=1e-6, act=act, scale=0.7)
    oh = o.double().view(19, H, dim)
    normed = oh / torch.sqrt((oh ** 2).mean(-1, keepdim=True) + 1e-6)
    normed = normed * (gain.double().view(1, 1, dim) if shared else gain.double().view(1, H, dim))
    z = gate.double().view(19, H, dim)
    want = normed * (z * torch.sigmoid(z) if act == "silu" else torch.sigmoid(z)) * 0.7
    assert (out.double().view(19, H, dim) - want).abs().max().item() < (2e-5 if dtype == torch.float32 else 4e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_activation(dtype):
    from sandyrt_b200.csrc import ops

    g = torch.Generator().manual_seed(3)
    both = (torch.randn(23, 2 * 77, generator=g) * 2).to(dtype).to(DEV)
    a, b = both[:, :77], both[:, 77:]
    out = torch.empty(23, 77, dtype=dtype, device=DEV)
    ops.glu(a, b, out, act="silu")
    # one rounding of the result: relative 2^-24 or 2^-9
    rel = 1e-6 if dtype == torch.float32 else 2 ** -8
    close = lambda got, want: bool(((got.double() - want).abs() <= rel * want.abs() + 1e-6).all())
    want = a.double() * torch.sigmoid(a.double()) * b.double()
    assert close(out, want)
    ops.glu(a, b, out, act="gelu_tanh")
    z = a.double()
    want = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))) * b.double()
    assert close(out, want)
