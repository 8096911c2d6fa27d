"""Each mechanism of the Vuvosun design alone: its kernels, driven the way the parts
drive them, against the one-mechanism functions of `plain_vuvosun.py`.  Inputs are made
so that a fault shows: one key's score stands far out at the places where a window, the
kept first tokens or a page ends, so a row that sees one key too many or too few is
wrong by the size of a value and not by rounding."""
from types import SimpleNamespace

import pytest
import torch

import plain_vuvosun as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: 3e-5, torch.bfloat16: 2e-2}


def rel(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    return float((got - ref).abs().max()) / max(float(ref.abs().max()), 1e-6)


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------------------
# residual streams
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("streams,width", [(1, 40), (3, 200), (8, 1100)])
def test_streams(dtype, streams, width):
    from crucible_b200.ops import streams as k
    rows, eps = 7, 1e-5
    table = torch.randn(50, width, device=DEV).to(dtype)
    gain = torch.rand(width, device=DEV) + 0.5
    ids = _i32([3, 49, 0, 7, 7, 21, 40])
    x = torch.empty(rows, streams, width, device=DEV)
    k.embed_norm(table, ids, gain, eps, x)
    x0 = plain.rms_norm(table.double().cpu()[ids.cpu().long()], gain.double().cpu(), eps)
    for s in range(streams):
        assert rel(x[:, s], x0) < 1e-6
    # streams that differ, then a read, a write, and a write with the next read
    x = torch.randn(rows, streams, width, device=DEV)
    w_in, w_out = torch.randn(streams, device=DEV), torch.randn(streams, device=DEV)
    w_mix = torch.randn(streams, streams, device=DEV)
    w_in2 = torch.randn(streams, device=DEV)
    y = torch.randn(rows, width, device=DEV)
    h = torch.empty(rows, width, device=DEV, dtype=dtype)
    k.read(x, w_in, gain, eps, h)
    old = [x[:, s].double().cpu() for s in range(streams)]
    seen = {}

    def y_of(normed):
        seen["h"] = normed
        return y.double().cpu()
    new = plain.hyper_sublayer(old, y_of, gain.double().cpu(), eps, w_in.double().cpu(),
                               w_mix.double().cpu(), w_out.double().cpu())
    assert rel(h, seen["h"]) < (1e-6 if dtype == torch.float32 else 6e-3)
    x2 = x.clone()
    k.write(x2, y, w_mix, w_out)
    h2 = torch.empty_like(h)
    k.write(x, y, w_mix, w_out, next_weights=w_in2, next_gain=gain, eps=eps, h=h2)
    assert torch.equal(x, x2)
    for s in range(streams):
        assert rel(x[:, s], new[s]) < 1e-6
    u2 = sum(w_in2.double().cpu()[s] * new[s] for s in range(streams))
    assert rel(h2, plain.rms_norm(u2, gain.double().cpu(), eps)) < (2e-6 if dtype == torch.float32 else 6e-3)
    out = torch.empty(3, width, device=DEV)
    k.sum_rows(x, _i32([6, 0, 3]), out)
    assert rel(out, sum(new)[[6, 0, 3]]) < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("ff", [52, 256, 3000])
def test_polynorm(dtype, ff):
    from crucible_b200 import ops
    z = (torch.randn(9, ff, device=DEV) * 1.5).to(dtype)
    coef = torch.tensor([0.7, -0.4, 0.25, 0.1], device=DEV)
    out = torch.empty_like(z)
    ops.polynorm(z, coef, 1e-5, out)
    ref = plain.polynorm(z.double().cpu(), coef.double().cpu(), 1e-5)
    assert rel(out, ref) < (2e-6 if dtype == torch.float32 else 6e-3)


# ---------------------------------------------------------------------------
# attention: the window's edges, the kept first tokens, pages, the sink
# ---------------------------------------------------------------------------

def _attention_case(dtype, H, G, D, E, R, window, keep, page, T, spikes, seed, sink_value=None):
    from crucible_b200.engine.context import CacheStorage
    g = torch.Generator().manual_seed(seed)
    width = H * D + G * D + G * E + H * E
    proj = torch.randn(T, width, generator=g) * 0.5
    q = proj[:, :H * D].view(T, H, D)
    k = proj[:, H * D:(H + G) * D].view(T, G, D)
    if spikes:
        # a feature that is not turned: every query looks for it, a few keys have it
        assert R < D
        q[:, :, D - 1] = 8.0
        k[:, :, D - 1] = 0.0
        for j in spikes:
            k[j, :, D - 1] = 8.0
    proj = proj.to(dtype)
    sinks = torch.randn(H, generator=g) if sink_value is None else torch.full((H,), float(sink_value))
    n_pages = -(-T // page) + 3
    perm = torch.randperm(n_pages, generator=g)[:-(-T // page)]        # scattered pages
    cache = CacheStorage(1, n_pages + 1, page, G, D, dtype, DEV, value_dim=E)
    table = torch.zeros(1, n_pages, dtype=torch.int32)
    table[0, :len(perm)] = perm.to(torch.int32)
    freq = (10000.0 ** (-2.0 * torch.arange(R // 2, dtype=torch.float32) / R)) if R else None
    # the plain result from the same (rounded) projections
    p64 = proj.double()
    pos = torch.arange(T)
    q64 = p64[:, :H * D].view(T, H, D)
    k64 = p64[:, H * D:(H + G) * D].view(T, G, D)
    v64 = p64[:, (H + G) * D:(H + G) * D + G * E].view(T, G, E)
    if R:
        q64 = plain.rotate_interleaved(q64, pos, 10000.0, R)
        k64 = plain.rotate_interleaved(k64, pos, 10000.0, R)
    scale = 0.25
    o = plain.attend(q64, k64, plain.rms_unit(v64, 1e-5), pos, sinks.double(), scale, window, keep)
    gate = torch.sigmoid(p64[:, -H * E:]).view(T, H, E)
    ref = (o * gate * 0.6).reshape(T, H * E)
    return SimpleNamespace(proj=proj.to(DEV), sinks=sinks.to(DEV), cache=cache, table=table.to(DEV),
                           freq=freq.to(DEV) if R else None, ref=ref, scale=scale,
                           dims=(H, G, D, E, R, window, keep))


def _run_attention(case, row_sets):
    """row_sets: lists of token indices, one kernel call each (a prompt's portion, or a
    single decoded token)."""
    from crucible_b200.ops import sink_attention as k
    H, G, D, E, R, window, keep = case.dims
    T = case.proj.shape[0]
    out = torch.zeros(T, H * E, device=DEV, dtype=case.proj.dtype)
    binding = SimpleNamespace(group=0, slot=0, write=True)
    for rows in row_sets:
        # one request that brings these rows (consecutive positions)
        assert rows == list(range(rows[0], rows[0] + len(rows)))
        ctx = SimpleNamespace(positions=_i32(rows), row_request=_i32([0] * len(rows)),
                              block_table=lambda g: case.table, req_row_start=_i32([0, len(rows)]),
                              req_first_pos=_i32([rows[0]]), n_requests=1,
                              host=SimpleNamespace(max_new_tokens=len(rows),
                                                   context_bucket=256 * (-(-(rows[-1] + 1) // 256))),
                              scratch=lambda name, shape, dtype: torch.empty(shape, device=DEV, dtype=dtype))
        proj = case.proj[rows].contiguous()
        act = torch.empty(len(rows), H * E, device=DEV, dtype=proj.dtype)
        k.rotate_norm_append(proj, case.freq, R, H, G, D, E, 1e-5, ctx, case.cache, binding)
        k.attention(proj[:, :H * D], proj[:, -H * E:], act, case.sinks, H, G, D, E, case.scale,
                    window, keep, 0.6, ctx, case.cache, binding)
        out[rows] = act
    return out


@pytest.mark.parametrize("dtype,E,tensor_cores", [(torch.float32, 16, False), (torch.bfloat16, 16, False),
                                                  (torch.bfloat16, 32, False), (torch.bfloat16, 32, True)])
@pytest.mark.parametrize("how", ["prompt", "portions", "decode"])
@pytest.mark.parametrize("window,keep,T", [(10, 3, 90), (70, 5, 300)])
def test_attention_sees_exactly_its_keys(dtype, E, tensor_cores, how, window, keep, T, monkeypatch):
    """E == 32 is the keys' size: the bfloat16 rows may then run on the tensor cores (64-key
    tiles: the longer case has tiles of kept tokens, tiles that are skipped, and rows whose
    window starts inside a tile)."""
    from crucible_b200.ops import sink_attention as k
    monkeypatch.setattr(k, "TENSOR_CORES", tensor_cores)
    page = 8
    # the last kept token and the first that is not; both sides of a page border; far back
    spikes = [keep - 1, keep, 7, 8, 40] + ([63, 64, 130] if T > 200 else [])
    case = _attention_case(dtype, 4, 2, 32, E, 16, window, keep, page, T, spikes, seed=1)
    if how == "prompt":
        sets = [list(range(T))]
    elif how == "portions":
        cuts = [0, 2, 9, 11, 12, 49, 51, 80] + ([150, 151, 290] if T > 200 else []) + [T]
        sets = [list(range(a, b)) for a, b in zip(cuts, cuts[1:])]
    else:
        sets = [list(range(5))] + [[t] for t in range(5, T)]
    out = _run_attention(case, sets)
    ref = case.ref
    # the rows just inside and just outside each spike's window, the kept ones far away
    for j in spikes:
        for i in (j, j + window - 1, j + window, T - 1):
            if i < T:
                assert rel(out[i], ref[i]) < TOL[dtype], (how, "key", j, "row", i)
    assert rel(out, ref) < TOL[dtype]
    # the test would see a window that is one off: the plain result itself changes there
    H, G, D, E, R, _, _ = case.dims
    assert (ref[keep + window] - ref[keep + window - 1]).abs().max() > 0.05


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_sink_counts_once_and_unscaled(dtype):
    # a sink as large as the scores: leaving it out, scaling it or counting it twice shows
    case = _attention_case(dtype, 2, 2, 16, 40, 16, None, 0, 16, 40, [], seed=2, sink_value=1.5)
    out = _run_attention(case, [list(range(40))])
    assert rel(out, case.ref) < TOL[dtype]
    without = _attention_case(dtype, 2, 2, 16, 40, 16, None, 0, 16, 40, [], seed=2, sink_value=-30.0)
    assert (without.ref - case.ref).abs().max() > 0.05


# ---------------------------------------------------------------------------
# matrix memories
# ---------------------------------------------------------------------------

def _state_ctx(portions, slots, state_bytes, n_slots=5):
    """One step in which request r brings portions[r] tokens and owns slot slots[r]."""
    starts = [0]
    for n in portions:
        starts.append(starts[-1] + n)
    row_request = [r for r, n in enumerate(portions) for _ in range(n)]
    return SimpleNamespace(row_request=_i32(row_request), req_row_start=_i32(starts),
                           req_state_slot=_i32(slots), n_requests=len(portions))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,E,taps", [(4, 2, 16, 24, 4), (2, 2, 40, 72, 3), (3, 1, 128, 32, 2),
                                          (1, 1, 136, 8, 1)])
def test_gated_delta_rule_in_portions(dtype, H, G, D, E, taps):
    """Two requests of unequal length in portions down to one and two tokens (shorter than
    the convolution's reach), in slots that are not in order, against the whole sequences."""
    from crucible_b200.ops import recurrent as k
    g = torch.Generator().manual_seed(H * 100 + D)
    lengths = [37, 11]
    C = 2 * G * D + H * E
    width = C + H * E
    projs = [(torch.randn(n, width, generator=g)).to(dtype) for n in lengths]
    gates = [torch.randn(n, 2 * H, generator=g) for n in lengths]
    conv_w = torch.rand(C, taps, generator=g) - 0.5
    a_log, dt_bias = torch.rand(H, generator=g) - 0.5, torch.rand(H, generator=g) - 0.5
    gain = torch.rand(E, generator=g) + 0.5
    s_bytes = 4 * H * D * E
    state = torch.zeros(5, s_bytes + 4 * (taps - 1) * C + 16, dtype=torch.uint8, device=DEV)
    state = state[:, :s_bytes + 4 * (taps - 1) * C]
    slots = [3, 1]
    schedule = [(2, 1), (1, 2), (1, 0), (9, 3), (16, 5), (8, 0)]         # tokens of each per step
    fed = [0, 0]
    outs = [torch.zeros(n, H * E, dtype=dtype) for n in lengths]
    for step in schedule:
        live = [r for r in range(2) if step[r] > 0]
        portions = [step[r] for r in live]
        ctx = _state_ctx(portions, [slots[r] for r in live], state.shape[1])
        proj = torch.cat([projs[r][fed[r]:fed[r] + step[r]] for r in live]).to(DEV)
        gt = torch.cat([gates[r][fed[r]:fed[r] + step[r]] for r in live]).to(DEV)
        t = proj.shape[0]
        qkv = torch.empty(t, C, device=DEV)
        beta, decay = torch.empty(t, H, device=DEV), torch.empty(t, H, device=DEV)
        o = torch.empty(t, H * E, device=DEV)
        act = torch.empty(t, H * E, device=DEV, dtype=dtype)
        k.delta_prepare(proj, conv_w.to(DEV), taps, gt, a_log.to(DEV), dt_bias.to(DEV), ctx, state,
                        s_bytes, qkv, beta, decay, H, G, D, E)
        k.conv_tail_update(proj, taps, C, ctx, state, s_bytes)
        k.matrix_memory(k.DELTA, qkv, 0, G * D, 2 * G * D, decay, beta, ctx, state, 0, 0, 0, o, H, G, D, E)
        k.head_norm_gate(o, gain.to(DEV), False, proj[:, C:], act, k.GATE_SILU, H, E, 1e-5, 1.1)
        at = 0
        for r in live:
            outs[r][fed[r]:fed[r] + step[r]] = act[at:at + step[r]].cpu()
            at += step[r]
            fed[r] += step[r]
    assert fed == lengths
    for r, n in enumerate(lengths):
        p = projs[r].double()
        x = plain.silu(plain.causal_conv(p[:, :C], conv_w.double()))
        q, kk = x[:, :G * D].view(n, G, D), x[:, G * D:2 * G * D].view(n, G, D)
        v = x[:, 2 * G * D:].view(n, H, E)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
        kk = kk / torch.sqrt((kk * kk).sum(-1, keepdim=True) + 1e-6)
        beta = torch.sigmoid(gates[r][:, :H].double())
        decay = torch.exp(-torch.exp(a_log.double())
                          * torch.nn.functional.softplus(gates[r][:, H:].double() + dt_bias.double()))
        ref = torch.zeros(n, H, E, dtype=torch.float64)
        for h in range(H):
            ref[:, h], _ = plain.delta_rule(q[:, h // (H // G)], kk[:, h // (H // G)], v[:, h],
                                            beta[:, h], decay[:, h])
        ref = plain.rms_unit(ref, 1e-5) * gain.double() * plain.silu(p[:, C:]).view(n, H, E) * 1.1
        assert rel(outs[r], ref.reshape(n, H * E)) < TOL[dtype], (r, H, G, D, E, taps)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,E", [(2, 16, 32), (3, 72, 40), (1, 256, 16)])
def test_mlstm_in_portions(dtype, H, D, E):
    from crucible_b200.ops import recurrent as k
    g = torch.Generator().manual_seed(D)
    n, cap = 45, 6.0
    C = 2 * H * D + H * E
    proj = (torch.randn(n, C + H * E, generator=g)).to(dtype)
    gates = torch.randn(n, 2 * H, generator=g) * 4.0                 # the cap is reached
    bias_i, bias_f = torch.randn(H, generator=g), torch.rand(H, generator=g) * 3.0
    gain = torch.rand(H * E, generator=g) + 0.5
    s_bytes, n_bytes = 4 * H * D * E, (4 * H * D + 15) // 16 * 16
    state = torch.zeros(3, s_bytes + n_bytes + 16, dtype=torch.uint8, device=DEV)
    out = torch.zeros(n, H * E, dtype=dtype)
    at = 0
    for count in [1, 2, 1, 17, 16, 8]:
        ctx = _state_ctx([count], [2], state.shape[1])
        p, gt = proj[at:at + count].to(DEV), gates[at:at + count].to(DEV)
        qkv = torch.empty(count, C, device=DEV)
        keep, inn = torch.empty(count, H, device=DEV), torch.empty(count, H, device=DEV)
        o = torch.empty(count, H * E, device=DEV)
        act = torch.empty(count, H * E, device=DEV, dtype=dtype)
        k.mlstm_prepare(p, gt, bias_i.to(DEV), bias_f.to(DEV), cap, qkv, keep, inn, H, D, E)
        k.matrix_memory(k.MLSTM, qkv, 0, H * D, 2 * H * D, keep, inn, ctx, state, 0, s_bytes,
                        s_bytes + n_bytes, o, H, H, D, E)
        k.head_norm_gate(o, gain.to(DEV), True, p[:, C:], act, k.GATE_SIGMOID, H, E, 1e-5, 1.0)
        out[at:at + count] = act.cpu()
        at += count
    assert at == n
    p = proj.double()
    q = p[:, :H * D].view(n, H, D) * D ** -0.5
    kk, v = p[:, H * D:2 * H * D].view(n, H, D), p[:, 2 * H * D:C].view(n, H, E)
    log_in, log_keep = plain.capped_log_gates(gates[:, :H].double() + bias_i.double(),
                                              gates[:, H:].double() + bias_f.double(), cap)
    ref = torch.zeros(n, H, E, dtype=torch.float64)
    for h in range(H):
        ref[:, h] = plain.matrix_memory(q[:, h], kk[:, h], v[:, h], log_in[:, h], log_keep[:, h])
    ref = plain.rms_unit(ref, 1e-5).reshape(n, H * E) * gain.double() * torch.sigmoid(p[:, C:])
    assert rel(out, ref) < TOL[dtype]
