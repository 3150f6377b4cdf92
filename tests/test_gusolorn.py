"""Gusolorn (pre-norm hybrid stack: mLSTM / windowed latent attention, dense or mixture-of-experts feed-forwards) against the plain
oracle in ``gusolorn_oracle.py``: every mechanism alone, prefill against token-by-token decoding, prompt portions down to two tokens,
ragged batches against each request alone, pages and state slots that are freed and used again, keys just inside / outside the window
and far away made visible by scaled weights, other sizes (top-k > 1, no shared expert, no window, column blocks), long decoding, and
greedy generation through the engine.

Runs on the CPU with the unfused ops; the ``gpu`` variants run the same cases on the sm_100a kernels in fp32 and bf16.
"""
import copy
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import gusolorn_oracle as oracle  # noqa: E402

from mlx_sharding_b200.config import ModelConfig  # noqa: E402
from mlx_sharding_b200.engine.core import LLMEngine  # noqa: E402
from mlx_sharding_b200.engine.sampler import SamplingParams  # noqa: E402
from mlx_sharding_b200.engine.trace import TraceSession  # noqa: E402
from mlx_sharding_b200.models import build_stage  # noqa: E402
from mlx_sharding_b200.parallel.pipeline import LocalPipeline, StageExecutor  # noqa: E402
from mlx_sharding_b200.utils.checkpoint import random_state_dict  # noqa: E402

DENSE = dict(ff=80, kind="dense")
MOE = dict(kind="moe", router=dict(experts=5, top=2), expert=dict(ff=24, limit=1.25), shared=dict(ff=40, limit=0.75))
MOE_NOSHARED = dict(kind="moe", router=dict(experts=3, top=3), expert=dict(ff=16, limit=0.5))
MLSTM = dict(type="mlstm", mixer=dict(dim=8, heads=3, vdim=12, gate_cap=2.5), mlp=None)
# value width 80 -> column blocks of 20 (four CTAs per head, each with its own copy of the normaliser state); dim != vdim
MLSTM_WIDE = dict(type="mlstm", mixer=dict(dim=24, heads=2, vdim=80, gate_cap=15.0), mlp=MOE)
ATTN = dict(type="latent_attention", mixer=dict(dim=24, heads=3, kv_rank=40, rot=dict(base=5000.0, dims=16), rot_dim=16, scale=0.2, vdim=8,
                                                mask=dict(size=9)), mlp=DENSE)
# reads layer 0's rows with other heads / sizes / window / scale of its own
ATTN_SHARED = dict(type="latent_attention", mixer=dict(dim=8, heads=5, kv_rank=40, rot=dict(base=5000.0, dims=16), rot_dim=16, scale=0.35, vdim=16,
                                                       mask=dict(size=21), kv_from=0), mlp=MOE)
# no window at all; kv_rank a multiple of 128 (the kernels' 16-byte path) and more heads than one CTA's warps
ATTN_FULL = dict(type="latent_attention", mixer=dict(dim=8, heads=9, kv_rank=128, rot=dict(base=300.0, dims=8), rot_dim=8, scale=0.3, vdim=8), mlp=None)
ATTN_W40 = dict(type="latent_attention", mixer=dict(dim=8, heads=2, kv_rank=24, rot=dict(base=100.0, dims=4), rot_dim=4, scale=0.5, vdim=8,
                                                    mask=dict(size=40)), mlp=MOE_NOSHARED)


def make_cfg(layers, width=48, vocab=96, eps=1e-3):
    return dict(architecture="Gusolorn", layers=copy.deepcopy(layers), norm=dict(eps=eps), vocab=vocab, width=width)


def make_model(cfgd, device="cpu", dtype=torch.float32, seed=3, edit=None):
    cfg = ModelConfig.from_dict(cfgd)
    sd = dict(random_state_dict(cfg, dtype=torch.bfloat16, seed=seed))
    if edit:
        edit(sd)
    model = build_stage(cfg, None, dtype, device).load_state({k: v.clone() for k, v in sd.items()})
    return model, sd


def session(model, pages=12, page_size=16, slots=4):
    return TraceSession(StageExecutor(model, pages, page_size, num_state_slots=slots + 1), (pages - 1) * page_size, slots)


def run_whole(model, tokens, **kw):
    s = session(model, **kw)
    return s.step([dict(id="a", tokens=tokens, want=list(range(len(tokens))))])


def toks(n, vocab=96, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def pick(cfgd, sd, dtype, make, seed, gap=0.08, tries=80):
    """Tokens ``make(seed)``.  In bf16 a router logit moves by about a hundredth, so a test that compares with exact arithmetic must
    not rest on a routing decision closer than that: other seeds are tried until the oracle's routing has no close call."""
    if dtype != torch.bfloat16:
        return make(seed)
    for i in range(tries):
        t = make(seed + 1000 * i)
        if oracle.min_router_gap(cfgd, sd, t) > gap:
            return t
    raise AssertionError("no sequence without a close routing call found")


def close(a, b, tol):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs().max().item() / max(1.0, b.abs().max().item())
    assert err < tol, f"relative error {err:.3e} >= {tol}"


def decode_after(model, t, n_prompt, **kw):
    s = session(model, **kw)
    got = [s.step([dict(id="r", tokens=t[:n_prompt], want=list(range(n_prompt)))])]
    got += [s.step([dict(id="r", tokens=[x], want=[0])]) for x in t[n_prompt:]]
    return torch.cat(got)


STACK = [ATTN, MLSTM, MLSTM_WIDE, ATTN_SHARED]
CASES = {"mlstm": [MLSTM], "mlstm_blocks_moe": [MLSTM_WIDE], "latent_window_dense": [ATTN], "latent_full": [ATTN_FULL],
         "latent_shared_rows": [ATTN, ATTN_SHARED], "latent_moe_noshared": [ATTN_W40], "stack": STACK}
DEVICES = [pytest.param("cpu", torch.float32, 2e-4, id="cpu"),
           pytest.param("cuda", torch.float32, 2e-4, id="b200-f32", marks=pytest.mark.gpu),
           pytest.param("cuda", torch.bfloat16, 6e-2, id="b200-bf16", marks=pytest.mark.gpu)]


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
@pytest.mark.parametrize("case", list(CASES))
def test_mechanism_against_oracle(case, device, dtype, tol):
    """Each mixer / feed-forward alone (and the mixed stack): whole prompt, every position; 45 tokens span three 16-token pages and
    run past the 9-, 21- and 40-token windows."""
    cfgd = make_cfg(CASES[case])
    model, sd = make_model(cfgd, device, dtype)
    t = pick(cfgd, sd, dtype, lambda s: toks(45, seed=s), 0)
    close(run_whole(model, t), oracle.forward(cfgd, sd, t), tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_first_tokens_and_single_token(device, dtype, tol):
    cfgd = make_cfg(STACK)
    model, sd = make_model(cfgd, device, dtype)
    for t in ([5], pick(cfgd, sd, dtype, lambda s: toks(2, seed=s), 4), pick(cfgd, sd, dtype, lambda s: toks(3, seed=s), 5)):
        close(run_whole(model, t), oracle.forward(cfgd, sd, t), tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
@pytest.mark.parametrize("portions", [[1] * 23, [2, 2, 2, 17], [16, 7], [15, 1, 1, 6], [3, 13, 7], [22, 1], [8, 9, 6]])
def test_portions_equal_whole(portions, device, dtype, tol):
    """Prefill against token-by-token decoding and prompts cut anywhere (page edge at 16, windows of 9 and 21, 2-token portions)."""
    cfgd = make_cfg(STACK)
    model, sd = make_model(cfgd, device, dtype)
    t = pick(cfgd, sd, dtype, lambda s: toks(sum(portions), seed=s), 1)
    want = oracle.forward(cfgd, sd, t)
    s, at, got = session(model), 0, []
    for n in portions:
        got.append(s.step([dict(id="r", tokens=t[at:at + n], want=list(range(n)))]))
        at += n
    close(torch.cat(got), want, tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_ragged_batch_and_reuse_of_pages_and_slots(device, dtype, tol):
    """Unequal requests in one batch (portions beside single tokens) equal each alone; a pool of 5 pages / 2 slots serves 4 requests
    one after another pair, so every page and slot is used again — by a request that must not see what the last one left."""
    cfgd = make_cfg(STACK)
    model, sd = make_model(cfgd, device, dtype)
    reqs = {n: pick(cfgd, sd, dtype, lambda s, L=L: toks(L, seed=s), 10 + i) for i, (n, L) in enumerate([("a", 30), ("b", 9), ("c", 17), ("d", 33)])}
    want = {n: oracle.forward(cfgd, sd, t) for n, t in reqs.items()}
    s = session(model, pages=6, page_size=16, slots=2)
    got = {n: [] for n in reqs}

    def step(parts, end=()):
        entries = [dict(id=n, tokens=reqs[n][lo:hi], want=list(range(hi - lo))) for n, lo, hi in parts]
        out = s.step(entries)
        at = 0
        for n, lo, hi in parts:
            got[n].append(out[at:at + hi - lo])
            at += hi - lo
        s.end(end)

    step([("a", 0, 13), ("b", 0, 1)])
    step([("a", 13, 14), ("b", 1, 8)])
    step([("b", 8, 9), ("a", 14, 29)], end=["b"])
    step([("a", 29, 30)], end=["a"])
    assert s.table.alloc.num_free == 5 and s.table.slots.num_free == 2
    step([("d", 0, 2), ("c", 0, 16)])
    step([("c", 16, 17), ("d", 2, 33)], end=["c", "d"])
    for n in reqs:
        close(torch.cat(got[n]), want[n], tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
@pytest.mark.parametrize("layer", ["own", "shared"])
def test_window_edges_show(layer, device, dtype, tol):
    """One token stands out among keys that are otherwise all alike.  It sits at position 20; with a window of W the query at 20 + W - 1 is the
    last that sees it and the one at 20 + W the first that does not: both in a prompt and decoded one by one, across a page edge.
    A window one shorter or longer would change those logits by far more than the tolerance."""
    layers = [ATTN, ATTN_SHARED] if layer == "shared" else [ATTN]
    W = layers[-1]["mixer"]["mask"]["size"]
    cfgd = make_cfg(layers)

    def make(seed):                     # from position 12 on one token is repeated, so every key in the edge queries' windows is the same
        t = [x if x != 95 else 3 for x in toks(20 + W + 6, seed=seed)]          # but the marked one at position 20
        t[12:] = [t[11]] * (len(t) - 12)
        t[20] = 95
        return t

    edit = lambda sd: sd[f"l{len(layers) - 1}.mix.q"].mul_(2.0)               # sharper attention

    model, sd = make_model(cfgd, device, dtype, edit=edit)
    t = pick(cfgd, sd, dtype, make, 7)
    want = oracle.forward(cfgd, sd, t)
    for delta in (-1, 1):               # a window one shorter / longer moves the edge position's logits far beyond the tolerance
        other = copy.deepcopy(cfgd)
        other["layers"][-1]["mixer"]["mask"]["size"] = W + delta
        edge = 20 + W - 1 + (1 if delta > 0 else 0)
        assert (oracle.forward(other, sd, t)[edge] - want[edge]).abs().max() > 2 * tol * want.abs().max()
    close(run_whole(model, t, pages=8), want, tol)
    close(decode_after(model, t, 18, pages=8), want, tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_far_key_without_window(device, dtype, tol):
    """No window: the key at position 1 is sought again 60 tokens later (four pages away), in a prompt and in decoding."""
    cfgd = make_cfg([ATTN_FULL])
    t = [x if x != 95 else 3 for x in toks(64, seed=8)]
    t[1] = t[62] = 95
    model, sd = make_model(cfgd, device, dtype, edit=lambda sd: sd["embed"][95].mul_(6.0))
    want = oracle.forward(cfgd, sd, t)
    close(run_whole(model, t, pages=8), want, tol)
    close(decode_after(model, t, 50, pages=8), want, tol)
    cut = copy.deepcopy(cfgd)
    cut["layers"][0]["mixer"]["mask"] = dict(size=32)
    assert (oracle.forward(cut, sd, t)[62] - want[62]).abs().max() > 1e-2


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_long_prompt_then_decode(device, dtype, tol):
    """A 290-token prompt (on the GPU a single long portion takes the matrix-product form of the attention, in blocks of queries that
    each see their own range of keys) with a 40-token window and with none, then single tokens; keys of a query split over CTAs."""
    cfgd = make_cfg([ATTN_W40, ATTN_FULL, MLSTM])
    model, sd = make_model(cfgd, device, dtype)
    t = toks(296, seed=9)
    want = oracle.forward(cfgd, sd, t)
    s = session(model, pages=21)
    rows = [0, 38, 39, 40, 41, 100, 127, 128, 289]
    got = [s.step([dict(id="r", tokens=t[:290], want=rows)])] + [s.step([dict(id="r", tokens=[x], want=[0])]) for x in t[290:]]
    close(torch.cat(got), torch.cat([want[rows], want[290:]]), tol * (3 if dtype == torch.bfloat16 else 1))


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_long_decode_keeps_state(device, dtype, tol):
    """150 single-token steps after a 3-token prompt: matrix memory, normaliser and running maximum carried exactly (a low gate cap
    and a high one), while the attention window slides on."""
    layers = [copy.deepcopy(MLSTM), MLSTM_WIDE, ATTN]
    layers[0]["mixer"]["gate_cap"] = 0.75
    cfgd = make_cfg(layers)
    model, sd = make_model(cfgd, device, dtype)
    t = pick(cfgd, sd, dtype, lambda s: toks(153 if dtype != torch.bfloat16 else 60, seed=s), 5, gap=0.05, tries=300)
    want = oracle.forward(cfgd, sd, t)
    close(decode_after(model, t, 3), want, tol * (3 if dtype == torch.bfloat16 else 1))


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_gates_that_saturate(device, dtype, tol):
    """Gate biases far out: the input gate at its cap while the forget gate closes (the running maximum jumps) and the reverse (the
    state decays towards exp(-m) in the denominator)."""
    def edit(sd):
        sd["l0.mix.i.b"][:] = torch.tensor([9.0, -9.0, 0.0])
        sd["l0.mix.f.b"][:] = torch.tensor([-9.0, 9.0, 0.0])

    cfgd = make_cfg([MLSTM])
    model, sd = make_model(cfgd, device, dtype, edit=edit)
    t = toks(40, seed=12)
    want = oracle.forward(cfgd, sd, t)
    close(run_whole(model, t), want, tol)
    close(decode_after(model, t, 7), want, tol)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 6e-2)])
def test_grouped_expert_gemm_sizes(dtype, tol):
    """Width and expert rows that are multiples of 128: bf16 takes the grouped tensor-core GEMM for the routed experts (a 40-token
    prompt: sorted rows; single tokens: one weight-row read per pair in exact mode)."""
    moe = dict(kind="moe", router=dict(experts=6, top=2), expert=dict(ff=128, limit=1.0), shared=dict(ff=32, limit=2.0))
    cfgd = make_cfg([dict(MLSTM, mlp=moe), dict(ATTN, mlp=moe)], width=128)
    model, sd = make_model(cfgd, "cuda", dtype)
    t = pick(cfgd, sd, dtype, lambda s: toks(44, seed=s), 2, gap=0.05, tries=300)
    want = oracle.forward(cfgd, sd, t)
    close(decode_after(model, t, 40), want, tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES[:2])
def test_greedy_generation_through_engine(device, dtype, tol):
    """The engine's scheduler, sampler and (on the GPU) captured decode graphs: two requests of unequal length, greedy tokens equal
    the oracle's argmax continuation."""
    cfgd = make_cfg(STACK)
    model, sd = make_model(cfgd, device, dtype)
    eng = LLMEngine(LocalPipeline([StageExecutor(model, 16, 16, num_state_slots=3)]), 16, 16, num_groups=1, max_prefill_tokens=11)
    prompts = [toks(19, seed=21), toks(4, seed=22)]
    rs = [eng.submit(p, SamplingParams(temperature=0.0), max_tokens=6) for p in prompts]
    eng.drain()
    for p, r in zip(prompts, rs):
        assert r.error is None
        seq = list(p)
        for _ in range(6):
            seq.append(int(oracle.forward(cfgd, sd, seq)[-1].argmax()))
        assert r.output == seq[len(p):]
    assert eng.table.slots.num_free == 2 and eng.table.alloc.num_free == 15


def test_config_reader_takes_every_size_from_the_file():
    cfg = ModelConfig.from_dict(make_cfg([ATTN, MLSTM_WIDE, ATTN_SHARED], width=40, vocab=50, eps=3e-3))
    assert (cfg.model_type, cfg.hidden_size, cfg.vocab_size, cfg.num_hidden_layers) == ("gusolorn", 40, 50, 3)
    assert cfg.rms_norm_eps == 3e-3 and cfg.layer_specs[0]["mixer"]["mask"]["size"] == 9 and cfg.layer_specs[2]["mixer"]["kv_from"] == 0
    assert cfg.layer_specs[1]["mlp"]["router"] == dict(experts=5, top=2) and cfg.layer_specs[1]["mixer"]["gate_cap"] == 15.0
    with pytest.raises(ValueError):
        ModelConfig.from_dict(make_cfg([dict(type="unknown", mixer=dict(heads=1), mlp=None)]))
    with pytest.raises(ValueError):      # kv_from must name an earlier layer that has rows of its own
        ModelConfig.from_dict(make_cfg([MLSTM, dict(ATTN_SHARED)]))
    bad = copy.deepcopy(ATTN_SHARED)
    bad["mixer"]["kv_rank"] = 48
    with pytest.raises(ValueError):
        ModelConfig.from_dict(make_cfg([ATTN, bad]))


def test_cache_layout_shares_rows_and_blocks_state():
    model, _ = make_model(make_cfg(STACK))
    kinds = [e[0] for e in model.cache_layout()]
    assert kinds == ["paged", "state", "state", "alias"]
    kv = StageExecutor(model, 4, 16, num_state_slots=3).kv
    assert kv.k[3] is kv.k[0] and kv.state[2]["n"].shape[1:] == (2, 4, 24) and kv.state[2]["m"].shape[1:] == (2, 4)
