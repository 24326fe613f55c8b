"""GPU parity of the three kernels, called through the C ABI, against the CPU oracle.

Tolerances (the stated parity targets): bf16 outputs <= 2e-2 max-abs and <= 1e-3 mean-abs; fp32 lse
<= 1e-3.  fp32 outputs computed from bf16 inputs meet the same bounds with margin."""
import math

import pytest
import torch

from oracle import ring_oracle as O

pytestmark = pytest.mark.gpu

MAX_ABS, MEAN_ABS, LSE_TOL = 2e-2, 1e-3, 1e-3


def _ops():
    from ditango_b200 import ops
    return ops


def _rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16)


def _check(out, lse, ref_out, ref_lse, what):
    eo = (out.float().cpu() - ref_out.float()).abs()
    el = (lse.cpu() - ref_lse).abs()
    el = el[torch.isfinite(ref_lse)]
    msg = f"{what}: out max {eo.max():.3e} mean {eo.mean():.3e}; lse max {el.max() if el.numel() else 0:.3e}"
    print(msg)
    assert el.numel() == 0 or el.max() <= LSE_TOL, msg
    assert eo.max() <= MAX_ABS and eo.mean() <= MEAN_ABS, msg


@pytest.mark.parametrize("B,Sq,Sk,H,D", [
    (1, 128, 128, 1, 64), (1, 128, 128, 1, 128), (1, 256, 384, 2, 128), (2, 300, 200, 3, 64),
    (1, 1, 1, 1, 64), (1, 63, 65, 2, 128), (1, 129, 127, 1, 64), (2, 257, 640, 2, 128),
    (1, 2222, 2222, 2, 64), (1, 1860, 3721, 3, 128),
])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_flash_partial_dense(B, Sq, Sk, H, D, out_dtype):
    ops = _ops()
    q, k, v = _rand((B, Sq, H, D), 1), _rand((B, Sk, H, D), 2), _rand((B, Sk, H, D), 3)
    ref_out, ref_lse = O.partial_attention(q, k, v, out_dtype=torch.float32)
    out, lse = ops.flash_partial(q.cuda(), k.cuda(), v.cuda(), out_dtype=out_dtype)
    assert ops.read_status() == 0
    assert out.dtype == out_dtype and lse.shape == (B, H, Sq)
    _check(out, lse, ref_out, ref_lse, f"dense B{B} Sq{Sq} Sk{Sk} H{H} D{D} {out_dtype}")


def test_flash_lse_layout_bsh_and_scale():
    ops = _ops()
    B, Sq, Sk, H, D = 2, 200, 333, 2, 64
    q, k, v = _rand((B, Sq, H, D), 4), _rand((B, Sk, H, D), 5), _rand((B, Sk, H, D), 6)
    ref_out, ref_lse = O.partial_attention(q, k, v, softmax_scale=0.3, out_dtype=torch.float32)
    out, lse = ops.flash_partial(q.cuda(), k.cuda(), v.cuda(), lse_layout=ops.LSE_BSH, softmax_scale=0.3)
    assert lse.shape == (B, Sq, H)
    _check(out, lse.transpose(1, 2), ref_out, ref_lse, "bsh layout")


def test_flash_large_logits_need_rescale():
    """Keys ordered so the running max keeps growing: exercises the lazy O rescale."""
    ops = _ops()
    B, Sq, Sk, H, D = 1, 256, 1024, 1, 64
    q = _rand((B, Sq, H, D), 7)
    k = _rand((B, Sk, H, D), 8) * torch.linspace(0.2, 6.0, Sk).view(1, Sk, 1, 1).to(torch.bfloat16)
    v = _rand((B, Sk, H, D), 9)
    ref_out, ref_lse = O.partial_attention(q, k, v, out_dtype=torch.float32)
    out, lse = ops.flash_partial(q.cuda(), k.cuda(), v.cuda())
    _check(out, lse, ref_out, ref_lse, "growing max")


def test_flash_accumulate_equals_attention_over_concatenated_keys():
    ops = _ops()
    B, Sq, H, D = 2, 300, 2, 128
    q = _rand((B, Sq, H, D), 10)
    ks = [_rand((B, n, H, D), 11 + i) for i, n in enumerate((256, 100, 513))]
    vs = [_rand((B, n, H, D), 21 + i) for i, n in enumerate((256, 100, 513))]
    ref_out, ref_lse = O.partial_attention(q, torch.cat(ks, 1), torch.cat(vs, 1), out_dtype=torch.float32)
    out = lse = None
    for i, (k, v) in enumerate(zip(ks, vs)):
        out, lse = ops.flash_partial(q.cuda(), k.cuda(), v.cuda(), out=out, lse=lse, accumulate=(i > 0))
    _check(out, lse, ref_out, ref_lse, "accumulate")


def test_flash_strided_views_of_packed_kv():
    """K and V living side by side in one receive slot: token stride 2*H*D."""
    ops = _ops()
    B, S, H, D = 1, 500, 2, 64
    q = _rand((B, S, H, D), 30).cuda()
    kv = _rand((B, S, 2, H, D), 31).cuda()
    k, v = kv[:, :, 0], kv[:, :, 1]
    ref_out, ref_lse = O.partial_attention(q.cpu(), k.cpu(), v.cpu(), out_dtype=torch.float32)
    out, lse = ops.flash_partial(q, k, v)
    _check(out, lse, ref_out, ref_lse, "strided kv")


def test_flash_packed_segments():
    ops = _ops()
    H, D = 2, 128
    cu_q = [0, 130, 130, 400, 448]       # second segment empty on the query side
    cu_k = [0, 200, 260, 260, 300]       # third segment has no keys
    q, k, v = _rand((448, H, D), 40), _rand((300, H, D), 41), _rand((300, H, D), 42)
    ref_out, ref_lse = O.partial_attention_varlen(q, k, v, cu_q, cu_k, out_dtype=torch.float32)
    cq = torch.tensor(cu_q, dtype=torch.int32).cuda()
    ck = torch.tensor(cu_k, dtype=torch.int32).cuda()
    out, lse = ops.flash_partial(q.cuda(), k.cuda(), v.cuda(), cu_seqlens_q=cq, cu_seqlens_k=ck,
                                 max_seqlen_q=270, max_seqlen_k=200)
    assert ops.read_status() == 0
    assert lse.shape == (H, 448)
    lse_c = lse.cpu()
    assert torch.isinf(lse_c[:, 130:400]).all() and (lse_c[:, 130:400] < 0).all()
    assert out.cpu()[130:400].abs().max() == 0
    _check(out, lse, ref_out, ref_lse, "packed")


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("n", [1, 2, 5, 9])
def test_merge_states_matches_pairwise_reference_merge(D, n):
    ops = _ops()
    B, S, H = 2, 77, 3
    g = torch.Generator().manual_seed(100 + n)
    states = []
    for i in range(n):
        o = torch.randn(B, S, H, D, generator=g)
        l = torch.randn(B, H, S, generator=g) * 3
        if i % 2:
            o = o.to(torch.bfloat16)
        states.append((o, l))
    ro = rl = None
    for o, l in states:
        ro, rl = O.merge_states(ro, rl, o, l)
    dev = []
    for i, (o, l) in enumerate(states):
        if i % 3 == 2:
            dev.append((o.cuda(), l.transpose(1, 2).contiguous().cuda(), ops.LSE_BSH))
        else:
            dev.append((o.cuda(), l.cuda(), ops.LSE_BHS))
    bf = torch.empty(B, S, H, D, dtype=torch.bfloat16, device="cuda")
    out, lse = ops.merge_states(dev, lse_out_layout=ops.LSE_BSH, out_bf16=bf)
    assert (out.cpu() - ro).abs().max() < 2e-5
    assert (lse.cpu() - rl.squeeze(-1)).abs().max() < 2e-5
    assert (bf.float().cpu() - ro).abs().max() < 2e-2
    out2, lse2 = ops.merge_states(dev, lse_out_layout=ops.LSE_BHS)
    assert torch.equal(lse2.transpose(1, 2), lse) and torch.equal(out2, out)


def test_merge_states_in_place_and_empty_rows():
    ops = _ops()
    B, S, H, D = 1, 50, 2, 64
    g = torch.Generator().manual_seed(7)
    o0, o1 = torch.randn(B, S, H, D, generator=g), torch.randn(B, S, H, D, generator=g)
    l0, l1 = torch.randn(B, S, H, generator=g), torch.randn(B, S, H, generator=g)
    l0[0, :10] = float("-inf")
    l1[0, 5:15] = float("-inf")
    o0[0, :10] = float("nan")            # an empty state's values must never leak
    ref = O.merge_states_exact([(torch.nan_to_num(o0), l0.transpose(1, 2)), (o1, l1.transpose(1, 2))])
    a, la = o0.cuda(), l0.cuda()
    ops.merge_states([(a, la, ops.LSE_BSH), (o1.cuda(), l1.cuda(), ops.LSE_BSH)], out=a, lse_out=la,
                     lse_out_layout=ops.LSE_BSH)
    got, gl = a.cpu(), la.cpu()
    assert torch.isinf(gl[0, 5:10]).all() and got[0, 5:10].abs().max() == 0
    fin = torch.isfinite(gl)
    assert (gl[fin] - ref[1].transpose(1, 2).float()[fin]).abs().max() < 1e-5
    assert (got - ref[0].float()).abs().max() < 1e-5


def test_copy_chunks_head_to_sequence_relayout():
    ops = _ops()
    N, B, S, H, D = 4, 2, 24, 8, 64
    Hn = H // N
    x = _rand((B, S, H, D), 50).cuda()
    y = _rand((B, S, H, D), 51).cuda()
    px, py = torch.empty(N, B, S, Hn, D, dtype=x.dtype, device="cuda"), torch.empty(N, B, S, Hn, D, dtype=x.dtype, device="cuda")
    C = Hn * D * 2
    ops.copy_chunks([(x, px), (y, py)], C, (N, B, S), (C, S * H * D * 2, H * D * 2), (B * S * C, S * C, C))
    ref = x.view(B, S, N, Hn, D).permute(2, 0, 1, 3, 4)
    assert torch.equal(px, ref.contiguous())
    assert torch.equal(py, y.view(B, S, N, Hn, D).permute(2, 0, 1, 3, 4).contiguous())


def test_rejected_arguments_raise():
    ops = _ops()
    from ditango_b200._capi import ExtensionError
    q = _rand((1, 8, 1, 32), 1).cuda()
    with pytest.raises(ExtensionError):
        ops.flash_partial(q, q, q)                      # head_dim 32 unsupported
    with pytest.raises(ExtensionError):
        ops.flash_partial(q.float(), q.float(), q.float())
    with pytest.raises(ExtensionError):
        ops.flash_partial(q.cpu(), q.cpu(), q.cpu())


@pytest.mark.parametrize("n", [1, 1000, 16384, 16385, 3_200_003])
def test_drift_accumulate_matches_reference_metric(n):
    ops = _ops()
    g = torch.Generator().manual_seed(n)
    prev = torch.randn(n, generator=g)
    cur = prev + 0.05 * torch.randn(n, generator=g)
    if n > 10:
        cur[3] = float("nan")
        prev[7] = float("nan")
    want = O.rel_l1(cur, prev)
    acc = torch.zeros(2, device="cuda")
    ops.drift_accumulate(cur.cuda(), prev.cuda(), acc[1:])
    ops.drift_accumulate(cur.cuda(), prev.cuda(), acc[1:])          # accumulates; scratch is reusable
    got = acc.cpu()
    assert got[0] == 0
    assert abs(got[1].item() - 2 * want) <= 2e-6 * max(1.0, abs(2 * want))


def test_drift_accumulate_special_cases():
    ops = _ops()
    n = 5000
    prev = torch.full((n,), 1e-9)
    cur = torch.randn(n, generator=torch.Generator().manual_seed(1))
    acc = torch.zeros(1, device="cuda")
    ops.drift_accumulate(cur.cuda(), prev.cuda(), acc)              # reference magnitude too small -> mean|cur|
    assert abs(acc.item() - O.rel_l1(cur, prev)) < 1e-6
    acc.zero_()
    ops.drift_accumulate(torch.full((n,), float("nan")).cuda(), prev.cuda(), acc)
    assert math.isinf(acc.item()) and O.rel_l1(torch.full((n,), float("nan")), prev) == float("inf")
    # an odd (4-byte aligned only) view takes the scalar path
    base = torch.randn(n + 1, generator=torch.Generator().manual_seed(2))
    acc.zero_()
    ops.drift_accumulate(base.cuda()[1:], (base * 1.1).cuda()[1:], acc)
    assert abs(acc.item() - O.rel_l1(base[1:], (base * 1.1)[1:])) < 1e-6
