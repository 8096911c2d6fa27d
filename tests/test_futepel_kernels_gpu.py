"""Each mechanism of the Futepel design alone: its part, driven over hand-made steps,
against the one-mechanism functions of `plain_futepel.py`.  Inputs are made so that a fault
shows: a few keys' scores stand far out (far back, at page borders, at the row's own
position and one beyond it), states and last tokens are left in slots that are used again."""
from types import SimpleNamespace

import pytest
import torch

import plain_futepel as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = {torch.float32: 3e-5, torch.bfloat16: 2.5e-2}


def rel(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    return float((got - ref).abs().max()) / max(float(ref.abs().max()), 1e-6)


def _i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


class Steps:
    """A stand-in for the engine around one part: state slots, one cache group with scattered
    pages, and the step's metadata for entries (slot, tokens brought)."""

    def __init__(self, dtype, state_bytes=0, cache_need=None, page=8, n_slots=4, max_tokens=512, seed=0):
        from crucible_b200.engine.context import CacheStorage, Scratch
        self.dtype, self.page = dtype, page
        self.scratch = Scratch(DEV)
        self.state = torch.zeros(n_slots, max(state_bytes, 16), dtype=torch.uint8, device=DEV)
        self.fed = [0] * n_slots
        self.storage = None
        if cache_need is not None:
            per = -(-max_tokens // page)
            self.storage = CacheStorage(1, n_slots * per + 1, page, cache_need.kv_heads, cache_need.head_dim,
                                        dtype, DEV, values_are_keys=cache_need.values_are_keys)
            g = torch.Generator().manual_seed(seed)
            perm = torch.randperm(n_slots * per, generator=g).to(torch.int32)
            self.tables = perm.view(n_slots, per)            # every slot's pages, scattered over the pool

    def free(self, slot):
        self.state[slot].zero_()
        self.fed[slot] = 0

    def ctx(self, entries, binding):
        from crucible_b200.engine.context import HostStep
        rows, req, starts, first, ctx_len, slots = [], [], [0], [], [], []
        for r, (slot, n) in enumerate(entries):
            rows += list(range(self.fed[slot], self.fed[slot] + n))
            req += [r] * n
            starts.append(starts[-1] + n)
            first.append(self.fed[slot])
            self.fed[slot] += n
            ctx_len.append(self.fed[slot])
            slots.append(slot)
        host = HostStep(request_ids=list(range(len(entries))), new_tokens=[n for _, n in entries],
                        first_pos=first, context_len=ctx_len, state_slots=slots)
        table = self.tables[slots].contiguous().to(DEV) if self.storage is not None else None
        state = self.state
        return SimpleNamespace(
            dtype=self.dtype, n_tokens=len(rows), n_requests=len(entries), host=host, positions=_i32(rows),
            row_request=_i32(req), req_row_start=_i32(starts), req_first_pos=_i32(first),
            req_context_len=_i32(ctx_len), req_state_slot=_i32(slots), device_tokens=None,
            scratch=self.scratch.get, cache=lambda group: self.storage, block_table=lambda group: table,
            state=lambda b: state[:, b.state_offset:b.state_offset + b.state_bytes] if b.state_bytes else None)


def _bind(part, dtype, seed, std=0.3, edit=None):
    """Random tensors for a part (rounded to bfloat16 so both dtypes and the plain model see
    the same numbers); returns them as float64 by local name for the plain functions."""
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for d in part.tensors():
        if d.init is not None:
            kind, a, b = d.init
            t = a + (b - a) * torch.rand(d.shape, generator=g) if kind == "uniform" else a + b * torch.randn(d.shape, generator=g)
        elif d.role == "vector":
            t = 1.0 + 0.2 * torch.randn(d.shape, generator=g)
        else:
            t = std * torch.randn(d.shape, generator=g)
        tensors[d.name] = t.to(torch.bfloat16).float()
    if edit is not None:
        edit(tensors)
        tensors = {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}
    part.bind({k: (v.to(dtype) if part_role(part, k) == "matrix" else v).to(DEV).contiguous()
               for k, v in tensors.items()}, dtype, torch.device(DEV))
    return {k: v.double() for k, v in tensors.items()}


def part_role(part, name):
    return next(d.role for d in part.tensors() if d.name == name)


def _binding(part, group=None):
    from crucible_b200.parts import LayerBinding
    return LayerBinding(group=group, slot=0, write=True, state_offset=0, state_bytes=int(part.state_bytes()))


def _run_mixer(part, steps, schedule, h_of, width):
    """Runs the schedule (a list of steps, each a list of (slot, n)); returns every slot's rows
    of the mixer's output in order."""
    binding = _binding(part, 0 if part.cache_need() is not None else None)
    out = {}
    for entries in schedule:
        ctx = steps.ctx(entries, binding)
        h = torch.cat([h_of[slot][steps.fed[slot] - n:steps.fed[slot]] for slot, n in entries], 0).to(steps.dtype).to(DEV)
        res = torch.zeros(h.shape[0], width, device=DEV)
        part.forward(ctx, h.contiguous(), res, binding)
        at = 0
        for slot, n in entries:
            out.setdefault(slot, []).append(res[at:at + n].clone())
            at += n
    torch.cuda.synchronize()
    return {slot: torch.cat(chunks, 0) for slot, chunks in out.items()}


def _cut(n, sizes):
    out, k = [], 0
    while n > 0:
        out.append(min(sizes[k % len(sizes)], n))
        n -= out[-1]
        k += 1
    return out


def _schedules(lengths):
    """Whole, token by token after a short start, and mixed portions with the slots out of
    order; `lengths`: slot -> tokens."""
    whole = [[(slot, n)] for slot, n in lengths.items()]
    single = []
    for slot, n in lengths.items():
        single += [[(slot, min(3, n))]] + [[(slot, 1)] for _ in range(n - min(3, n))]
    cuts = {slot: _cut(n, [2, 5, 1, 17, 3]) for slot, n in lengths.items()}
    mixed = []
    while any(cuts.values()):
        mixed.append([(slot, c.pop(0)) for slot, c in sorted(cuts.items(), reverse=True) if c])
    return {"whole": whole, "single": single, "mixed": mixed}


def _check_mixer(kind_spec, plain_fn, dtype, lengths, page=8, edit=None, h_edit=None, tol=None, std=0.3):
    from crucible_b200.parts import MIXERS
    part = MIXERS.build(kind_spec.kind, kind_spec)
    w = _bind(part, dtype, seed=5, std=std, edit=edit)
    g = torch.Generator().manual_seed(9)
    h_of = {slot: torch.randn(n, kind_spec.width, generator=g).to(torch.bfloat16).float() for slot, n in lengths.items()}
    if h_edit is not None:
        for h in h_of.values():
            h_edit(h)
        h_of = {slot: h.to(torch.bfloat16).float() for slot, h in h_of.items()}
    ref = {slot: plain_fn(h.double(), w) for slot, h in h_of.items()}
    results = {}
    for label, schedule in _schedules(lengths).items():
        steps = Steps(dtype, state_bytes=int(part.state_bytes()), cache_need=part.cache_need(), page=page,
                      n_slots=max(lengths) + 1, max_tokens=max(lengths.values()) + page)
        got = _run_mixer(part, steps, schedule, h_of, kind_spec.width)
        for slot in lengths:
            e = rel(got[slot], ref[slot])
            assert e < (tol or TOL[dtype]), (label, slot, e)
        results[label] = got
    if dtype == torch.float32:
        for label in ("single", "mixed"):
            for slot in lengths:
                assert torch.equal(results[label][slot], results["whole"][slot]), (label, slot)
    return part


# ---------------------------------------------------------------------------
# embedding: scale, hashed bigram rows with the last token kept between steps, positions
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("bigram,positions", [((97, 31, 5), 64), ((1009, 2147483647, 65537), None), (None, 40)])
def test_hashed_embedding(dtype, bigram, positions):
    from crucible_b200.config.model_config import EndSpec
    from crucible_b200.parts import EMBEDDINGS, LayerBinding
    vocab, width = 150, 48
    part = EMBEDDINGS.build("token_hashed_positions",
                            EndSpec("token_hashed_positions", (("scale", 3.0), ("bigram", bigram),
                                                               ("max_positions", positions))), vocab, width)
    w = _bind(part, dtype, seed=2)
    names = {"table": "embed", "bigram": "bigram", "positions": "pos"}
    pw = {names[k]: v for k, v in w.items()}
    cfg = {"scale": 3.0, "bigram": dict(zip(("buckets", "mul_prev", "mul_cur"), bigram)) if bigram else None}
    part.state_binding = LayerBinding(state_offset=0, state_bytes=part.state_bytes())
    g = torch.Generator().manual_seed(1)
    tokens = {slot: torch.randint(0, vocab, (n,), generator=g).tolist() for slot, n in {0: 23, 2: 9, 3: 31}.items()}
    steps = Steps(dtype, state_bytes=16)
    for again in range(2):                       # the second time the slots hold what the first left
        got = {}
        cuts = {slot: _cut(len(t), [1, 4, 2, 9]) for slot, t in tokens.items()}
        while any(cuts.values()):
            entries = [(slot, c.pop(0)) for slot, c in sorted(cuts.items(), reverse=True) if c]
            ctx = steps.ctx(entries, None)
            ids = _i32([t for slot, n in entries for t in tokens[slot][steps.fed[slot] - n:steps.fed[slot]]])
            x = part.forward(ctx, ids)
            at = 0
            for slot, n in entries:
                got.setdefault(slot, []).append(x[at:at + n].clone())
                at += n
        for slot, t in tokens.items():
            assert rel(torch.cat(got[slot], 0), plain.embed(t, pw, cfg)) < 1e-6, (again, slot)
            steps.free(slot)


# ---------------------------------------------------------------------------
# the recurrent mixers: portions down to one token, slots out of order, bit-equal cuts
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,width,rank", [(2, 16, 40, 5), (3, 64, 128, 16), (1, 36, 24, 8)])
def test_wkv(dtype, heads, dim, width, rank):
    from crucible_b200.config.model_config import MixerSpec
    spec = MixerSpec(kind="wkv", width=width, n_heads=heads, n_kv_heads=heads, head_dim=dim,
                     extra=(("norm_eps", 1e-5), ("decay_rank", rank)))
    cfg = {"heads": heads, "dim": dim}
    _check_mixer(spec, lambda h, w: plain.wkv_mixer(h, w, cfg, 1e-5), dtype, {0: 45, 2: 7, 3: 1})


def test_wkv_decay_and_bonus_alone():
    """The recurrence by itself against the plain loop, with decays near 0 and near 1."""
    from crucible_b200.ops import recurrent as k
    T, H, D = 37, 2, 24
    g = torch.Generator().manual_seed(3)
    r, kk, v = (torch.randn(T, H * D, generator=g) for _ in range(3))
    w = torch.rand(T, H * D, generator=g) ** 3
    w[5] = 0.999
    w[6] = 1e-4
    u = torch.randn(H, D, generator=g)
    qkv = torch.cat([r, kk, v, w], 1).to(DEV).contiguous()
    steps = Steps(torch.float32, state_bytes=4 * H * D * D)
    from crucible_b200.parts import LayerBinding
    b = LayerBinding(state_offset=0, state_bytes=4 * H * D * D)
    out = torch.zeros(T, H * D, device=DEV)
    at = 0
    for n in _cut(T, [1, 16, 3, 17]):
        ctx = steps.ctx([(1, n)], b)
        o = torch.zeros(n, H * D, device=DEV)
        k.matrix_memory(k.WKV, qkv[at:at + n].contiguous(), 0, H * D, 2 * H * D, None, None, ctx, ctx.state(b),
                        0, 0, 0, o, H, H, D, D, w_off=3 * H * D, per_head=u.to(DEV).contiguous())
        out[at:at + n] = o
        at += n
    ref = plain.wkv_recurrence(*(x.double().view(T, H, D) for x in (r, kk, v, w)), u.double())
    assert rel(out, ref.reshape(T, H * D)) < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,vdim,state,groups,conv,parts,width",
                         [(4, 16, 24, 2, 3, 2, 40), (2, 64, 64, 1, 4, 1, 128), (3, 20, 12, 3, 1, 3, 24),
                          (1, 8, 130, 1, 2, 1, 16)])
def test_mamba2(dtype, heads, vdim, state, groups, conv, parts, width):
    from crucible_b200.config.model_config import MixerSpec
    spec = MixerSpec(kind="mamba2", width=width, n_heads=heads, n_kv_heads=groups, head_dim=state,
                     extra=(("value_dim", vdim), ("conv_taps", conv), ("norm_groups", parts), ("norm_eps", 1e-5)))
    cfg = {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": parts}
    _check_mixer(spec, lambda h, w: plain.mamba2_mixer(h, w, cfg, 1e-5), dtype, {0: 45, 2: 7, 3: 1})


# ---------------------------------------------------------------------------
# latent attention: keys far back, at page borders, at the row's own position
# ---------------------------------------------------------------------------

def _latent_spec(heads, dim, rot, vdim, rank, width, scaling, turned=None):
    from crucible_b200.config.model_config import MixerSpec, PositionSpec
    position = PositionSpec(kind="rope_yarn", rotary_dim=turned or rot, theta=1000.0, max_positions=0,
                            scaling=tuple(scaling.items()) if scaling else None)
    return MixerSpec(kind="latent_attention", width=width, n_heads=heads, n_kv_heads=1, head_dim=dim,
                     softmax_scale=0.25, position=position,
                     extra=(("rot_dim", rot), ("value_dim", vdim), ("kv_rank", rank), ("norm_eps", 1e-5),
                            ("gate", True)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,rot,vdim,rank,width,page,scaling",
                         [(2, 24, 8, 16, 40, 48, 8, {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}),
                          (4, 32, 32, 32, 96, 64, 16, None),            # rows of 128: tensor cores in bfloat16
                          (2, 16, 16, 16, 48, 32, 8, None),             # rows of 64
                          (3, 10, 6, 14, 21, 40, 4, {"factor": 2.0, "original": 32, "fast": 4.0, "slow": 1.0})])
def test_latent_attention_finds_marked_keys(dtype, heads, dim, rot, vdim, rank, width, page, scaling):
    """Feature 0 of the input is 1 for every token and feature 1 is large for a few marked
    tokens; latent channel 0 reads feature 1 alone, every head's key channel 0 reads latent
    channel 0 and its query channel 0 reads feature 0.  So every row's softmax is held by the
    marked keys it may see: one far back, those around page borders, and the row itself."""
    marked = [2, page - 1, page, 3 * page - 1, 3 * page, 150, 263]

    def edit(t):
        t["dkv"][0] = 0.0
        t["dkv"][0, 1] = 1.0
        t["dkv"][1:, 1] = 0.0
        t["uk"].view(heads, dim, rank)[:, 0, :] = 0.0
        t["uk"].view(heads, dim, rank)[:, 0, 0] = 2.0
        t["q"].view(heads, dim + rot, width)[:, 0, :] = 0.0
        t["q"].view(heads, dim + rot, width)[:, 0, 0] = 6.0

    def h_edit(h):
        h[:, 0] = 1.0
        h[:, 1] = 0.0
        for j in marked:
            if j < h.shape[0]:
                h[j, 1] = 4.0

    spec = _latent_spec(heads, dim, rot, vdim, rank, width, scaling)
    cfg = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "scale": 0.25,
           "rot": {"base": 1000.0, "dims": rot, "scaling": scaling}}

    def ref(h, w):
        return plain.latent_attention(h, w, cfg, 1e-5, torch.arange(h.shape[0]))
    _check_mixer(spec, ref, dtype, {0: 270, 1: 3 * page + 1, 3: 2}, page=page, edit=edit, h_edit=h_edit, std=0.1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_turns_a_part_of_the_rotated_features(dtype):
    heads, dim, rot, vdim, rank, width, turned = 2, 12, 12, 8, 20, 32, 8
    spec = _latent_spec(heads, dim, rot, vdim, rank, width, None, turned=turned)
    cfg = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "scale": 0.25,
           "rot": {"base": 1000.0, "dims": turned, "scaling": None}}
    _check_mixer(spec, lambda h, w: plain.latent_attention(h, w, cfg, 1e-5, torch.arange(h.shape[0])), dtype,
                 {0: 40, 1: 9}, page=8)


def test_latent_attention_marked_keys_matter():
    """The construction above does what it says: without the far key the plain result moves."""
    heads, dim, rot, vdim, rank, width = 2, 24, 8, 16, 40, 48
    cfg = {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": rank, "scale": 0.25,
           "rot": {"base": 1000.0, "dims": rot, "scaling": None}}
    g = torch.Generator().manual_seed(0)
    w = {"q": torch.randn(heads * (dim + rot), width, generator=g) * 0.1, "dkv": torch.randn(rank + rot, width, generator=g) * 0.1,
         "dkv.norm": torch.ones(rank), "uk": torch.randn(heads * dim, rank, generator=g) * 0.1,
         "uv": torch.randn(heads * vdim, rank, generator=g) * 0.1, "g": torch.randn(heads, width, generator=g),
         "o": torch.randn(width, heads * vdim, generator=g) * 0.1}
    w["dkv"][0] = 0.0; w["dkv"][0, 1] = 1.0; w["dkv"][1:, 1] = 0.0
    w["uk"].view(heads, dim, rank)[:, 0, :] = 0.0; w["uk"].view(heads, dim, rank)[:, 0, 0] = 2.0
    w["q"].view(heads, dim + rot, width)[:, 0, :] = 0.0; w["q"].view(heads, dim + rot, width)[:, 0, 0] = 6.0
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(200, width, generator=g).double()
    h[:, 0] = 1.0; h[:, 1] = 0.0; h[2, 1] = 4.0
    full = plain.latent_attention(h, w, cfg, 1e-5, torch.arange(200))
    cut = plain.latent_attention(h[3:], w, cfg, 1e-5, torch.arange(3, 200))
    assert rel(cut[-1:], full[-1:]) > 0.2


# ---------------------------------------------------------------------------
# feed-forwards
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,ff,shared,width,rows", [(6, 2, 40, 24, 48, 77), (4, 1, 20, 0, 24, 5),
                                                              (8, 8, 64, 64, 128, 200), (40, 5, 12, 0, 36, 300)])
def test_mixture_of_experts(dtype, experts, top, ff, shared, width, rows):
    from crucible_b200.config.model_config import FeedForwardSpec
    from crucible_b200.parts import FEED_FORWARDS
    spec = FeedForwardSpec(kind="moe", width=width, intermediate=ff,
                           extra=(("experts", experts), ("top", top), ("shared_intermediate", shared or None)))
    part = FEED_FORWARDS.build("moe", spec)
    w = _bind(part, dtype, seed=4)
    cfg = {"router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    g = torch.Generator().manual_seed(8)
    h = torch.randn(rows, width, generator=g).to(torch.bfloat16).float()
    ref = plain.moe_ff(h.double(), w, cfg)
    steps = Steps(dtype)
    ctx = steps.ctx([(0, rows)], None)
    res = torch.zeros(rows, width, device=DEV)
    part.forward(ctx, h.to(dtype).to(DEV), res)
    assert rel(res, ref) < TOL[dtype]
    # a token's result does not depend on what else is in the step
    few = [0, rows // 2, rows - 1]
    ctx = Steps(dtype).ctx([(0, len(few))], None)
    alone = torch.zeros(len(few), width, device=DEV)
    part.forward(ctx, h[few].to(dtype).to(DEV), alone)
    if dtype == torch.float32:
        assert torch.equal(alone, res[few])
    else:
        assert rel(alone, ref[few]) < TOL[dtype]


def test_routing_takes_the_lower_index_on_equal_logits():
    from crucible_b200.ops import moe as k
    logits = torch.tensor([[0.5, 2.0, 2.0, -1.0, 2.0], [3.0, 1.0, 0.0, 3.0, -2.0]], device=DEV)
    top, n = 2, 5
    tiles = k.max_tiles(2, top, n)
    idx, place, order = (torch.zeros(4, dtype=torch.int32, device=DEV) for _ in range(3))
    weight = torch.zeros(4, device=DEV)
    count = torch.zeros(n, dtype=torch.int32, device=DEV)
    plan = torch.zeros(k.plan_ints(n, tiles), dtype=torch.int32, device=DEV)
    k.route(logits, top, idx, weight, place, count, plan, tiles, order)
    assert idx.tolist() == [1, 2, 0, 3]
    assert torch.allclose(weight.cpu(), torch.tensor([0.5, 0.5, 0.5, 0.5]))
    assert count.tolist() == [0] * n                     # left ready for the next step
    assert sorted(order.tolist()) == [0, 1, 2, 3]
    assert plan[0].item() == 4                           # four experts in use, one tile each


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dense_feed_forward_and_activations(dtype):
    from crucible_b200 import ops
    from crucible_b200.config.model_config import FeedForwardSpec
    from crucible_b200.parts import FEED_FORWARDS
    part = FEED_FORWARDS.build("dense_act", FeedForwardSpec(kind="dense_act", width=40, intermediate=72,
                                                            extra=(("activation", "relu2"),)))
    w = _bind(part, dtype, seed=6)
    h = torch.randn(19, 40).to(torch.bfloat16).float()
    res = torch.zeros(19, 40, device=DEV)
    part.forward(Steps(dtype).ctx([(0, 19)], None), h.to(dtype).to(DEV), res)
    assert rel(res, plain.relu2_ff(h.double(), w)) < TOL[dtype]
    z = (torch.randn(7, 33, device=DEV) * 2).to(dtype)
    out = torch.empty_like(z)
    z64 = z.double().cpu()
    for kind, ref in (("relu2", torch.relu(z64) ** 2), ("tanh", torch.tanh(z64)), ("silu", plain.silu(z64))):
        ops.activation(kind, z, out)
        assert rel(out, ref) < (2e-6 if dtype == torch.float32 else 6e-3), kind


def test_gate_then_norm_in_parts():
    from crucible_b200.ops import recurrent as k
    y = torch.randn(11, 96, device=DEV)
    gate = torch.randn(11, 96, device=DEV)
    gain = torch.rand(96, device=DEV) + 0.5
    for parts in (1, 2, 6):
        out = torch.empty(11, 96, device=DEV)
        k.gate_group_norm(y, gate, gain, out, parts, 1e-5)
        v = (y.double() * plain.silu(gate.double())).cpu()
        ref = plain.rms_unit(v.view(11, parts, 96 // parts), 1e-5).reshape(11, 96) * gain.double().cpu()
        assert rel(out, ref) < 2e-6
