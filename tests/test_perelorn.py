"""Perelorn (hybrid stack) against the plain oracle in ``perelorn_oracle.py``: every mechanism alone, prefill against token-by-token
decoding, prompt portions down to two tokens, ragged batches against each request alone, pages and state slots that are freed and
used again, far keys / sinks made visible by scaled weights, odd sizes, and greedy generation through the engine.

Runs on the CPU with the unfused ops; the ``gpu`` variants run the same cases on the sm_100a kernels in fp32 and bf16.
"""
import copy
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import perelorn_oracle as oracle  # noqa: E402

from mlx_sharding_b200.config import ModelConfig  # noqa: E402
from mlx_sharding_b200.engine.core import LLMEngine  # noqa: E402
from mlx_sharding_b200.engine.sampler import SamplingParams  # noqa: E402
from mlx_sharding_b200.engine.trace import TraceSession  # noqa: E402
from mlx_sharding_b200.models import build_stage  # noqa: E402
from mlx_sharding_b200.parallel.pipeline import LocalPipeline, StageExecutor  # noqa: E402
from mlx_sharding_b200.utils.checkpoint import random_state_dict  # noqa: E402

MAMBA = dict(type="mamba2", mixer=dict(conv=4, groups=1, heads=3, norm_groups=3, state=8, vdim=16), mlp=None)
MAMBA_G = dict(type="mamba2", mixer=dict(conv=2, groups=2, heads=4, norm_groups=1, state=24, vdim=8), mlp=dict(ff=96, kind="dense"))
ATTN = dict(type="latent_attention", mixer=dict(dim=24, heads=3, kv_rank=40, q_rank=32, rot=dict(base=5000.0, dims=16), rot_dim=16,
                                                scale=0.2, vdim=8), mlp=dict(ff=80, kind="dense"))
# kv_rank a multiple of 128 (the kernels' 16-byte path) and more heads than one CTA's warps
ATTN_WIDE = dict(type="latent_attention", mixer=dict(dim=8, heads=9, kv_rank=256, q_rank=16, rot=dict(base=300.0, dims=8), rot_dim=8,
                                                     scale=0.3, vdim=8), mlp=None)
# latent wider than 512: the kernels' second register budget, with and without the 16-byte path
ATTN_XL = dict(type="latent_attention", mixer=dict(dim=8, heads=2, kv_rank=640, q_rank=8, rot=dict(base=50.0, dims=4), rot_dim=4,
                                                   scale=0.2, vdim=8), mlp=None)
ATTN_XL_ODD = dict(type="latent_attention", mixer=dict(dim=8, heads=2, kv_rank=522, q_rank=8, rot=dict(base=50.0, dims=6), rot_dim=6,
                                                       scale=0.2, vdim=8), mlp=None)
LIGHT = dict(type="lightning", mixer=dict(decay=[0.5, 0.97], dim=16, heads=2, vdim=24), mlp=None)


def make_cfg(layers, width=48, vocab=96, side=8, logit_scale=1.5, eps=1e-4):
    d = dict(architecture="Perelorn", layers=copy.deepcopy(layers), logit_scale=logit_scale, norm=dict(eps=eps), vocab=vocab, width=width)
    if side:
        d["token_side"] = dict(dim=side)
    return d


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


def close(a, b, tol):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs().max().item() / max(1.0, b.abs().max().item())
    assert err < tol, f"relative error {err:.3e} >= {tol}"


CASES = {"latent_xl": [ATTN_XL, ATTN_XL_ODD], "latent_wide": [ATTN_WIDE], "mamba2": [MAMBA], "mamba2_groups": [MAMBA_G], "latent": [ATTN], "lightning": [LIGHT], "stack": [MAMBA, ATTN, LIGHT, MAMBA_G, ATTN]}
DEVICES = [pytest.param("cpu", torch.float32, 2e-4, id="cpu"),
           pytest.param("cuda", torch.float32, 2e-4, id="b200-f32", marks=pytest.mark.gpu),
           pytest.param("cuda", torch.bfloat16, 6e-2, id="b200-bf16", marks=pytest.mark.gpu)]


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
@pytest.mark.parametrize("case", list(CASES))
def test_mechanism_against_oracle(case, device, dtype, tol):
    """Each mixer alone (and the mixed stack): whole prompt, every position; 37 tokens span three 16-token pages."""
    cfgd = make_cfg(CASES[case])
    model, sd = make_model(cfgd, device, dtype)
    t = toks(37)
    close(run_whole(model, t), oracle.forward(cfgd, sd, t), tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_no_side_input_no_scale_single_token(device, dtype, tol):
    cfgd = make_cfg([LIGHT, ATTN, MAMBA], side=0, logit_scale=1.0)
    model, sd = make_model(cfgd, device, dtype)
    for t in ([5], toks(2, seed=4)):
        close(run_whole(model, t), oracle.forward(cfgd, sd, t), tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
@pytest.mark.parametrize("portions", [[1] * 21, [2, 2, 2, 15], [16, 5], [15, 1, 1, 4], [3, 13, 5], [20, 1]])
def test_portions_equal_whole(portions, device, dtype, tol):
    """Prefill against token-by-token decoding and prompts cut anywhere (page edge at 16, conv window of 4, 2-token portions)."""
    cfgd = make_cfg(CASES["stack"])
    model, sd = make_model(cfgd, device, dtype)
    t = toks(sum(portions), seed=1)
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
    cfgd = make_cfg(CASES["stack"])
    model, sd = make_model(cfgd, device, dtype)
    reqs = {n: toks(L, seed=10 + i) for i, (n, L) in enumerate([("a", 30), ("b", 9), ("c", 17), ("d", 33)])}
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
def test_far_key_and_sink_show(device, dtype, tol):
    """One score made to stand out: the key at position 1 is sought again 60 tokens later (four pages away); and a sink so large that
    leaving it out of the denominator changes every output."""
    cfgd = make_cfg([ATTN], side=0)
    t = toks(64, seed=7)
    t[1] = t[62] = 95          # same token -> same latent; query of position 62 looks for it

    def edit(sd):
        sd["embed"][95] *= 6.0
        sd["l0.mix.sink"][:] = torch.tensor([4.0, -3.0, 0.5])

    model, sd = make_model(cfgd, device, dtype, edit=edit)
    want = oracle.forward(cfgd, sd, t)
    close(run_whole(model, t, pages=8), want, tol)
    s = session(model, pages=8)
    s.step([dict(id="r", tokens=t[:50], want=[])])
    got = [s.step([dict(id="r", tokens=[x], want=[0])]) for x in t[50:]]
    close(torch.cat(got), want[50:], tol)
    nosink = copy.deepcopy(sd)
    nosink["l0.mix.sink"][:] = -1e4
    assert (oracle.forward(cfgd, nosink, t) - want).abs().max() > 1e-2


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_long_context_decode(device, dtype, tol):
    """A 290-token prompt (the attention of a single long portion takes the matrix-product form on the GPU) and then single tokens
    whose keys are split over several CTAs and merged with the sink."""
    cfgd = make_cfg([ATTN_WIDE, LIGHT], side=0)
    model, sd = make_model(cfgd, device, dtype, edit=lambda sd: sd["l0.mix.sink"].copy_(torch.linspace(-2, 3, 9)))
    t = toks(296, seed=9)
    want = oracle.forward(cfgd, sd, t)
    s = session(model, pages=21)
    got = [s.step([dict(id="r", tokens=t[:290], want=[0, 100, 289])])] + [s.step([dict(id="r", tokens=[x], want=[0])]) for x in t[290:]]
    close(torch.cat(got), torch.cat([want[[0, 100, 289]], want[290:]]), tol)


@pytest.mark.parametrize("device,dtype,tol", DEVICES)
def test_long_decode_keeps_state(device, dtype, tol):
    """150 single-token steps after a 3-token prompt: recurrent state and conv history carried exactly; slow and fast decays."""
    layers = [copy.deepcopy(LIGHT), MAMBA]
    layers[0]["mixer"]["decay"] = [0.999, 0.3]
    cfgd = make_cfg(layers)
    model, sd = make_model(cfgd, device, dtype)
    t = toks(153, seed=5)
    want = oracle.forward(cfgd, sd, t)
    s = session(model, pages=12)
    got = [s.step([dict(id="r", tokens=t[:3], want=[0, 1, 2])])] + [s.step([dict(id="r", tokens=[x], want=[0])]) for x in t[3:]]
    close(torch.cat(got), want, tol * (3 if dtype == torch.bfloat16 else 1))


@pytest.mark.parametrize("device,dtype,tol", DEVICES[:2])
def test_greedy_generation_through_engine(device, dtype, tol):
    """The engine's scheduler, sampler and (on the GPU) captured decode graphs: two requests of unequal length, greedy tokens equal
    the oracle's argmax continuation."""
    cfgd = make_cfg(CASES["stack"])
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
    cfg = ModelConfig.from_dict(make_cfg([MAMBA, ATTN], width=40, vocab=50, side=4, eps=3e-3, logit_scale=0.25))
    assert (cfg.model_type, cfg.hidden_size, cfg.vocab_size, cfg.num_hidden_layers) == ("perelorn", 40, 50, 2)
    assert cfg.rms_norm_eps == 3e-3 and cfg.logit_scale == 0.25 and cfg.token_side_dim == 4
    assert cfg.layer_specs[1]["mixer"]["kv_rank"] == 40 and cfg.layer_specs[0]["mlp"] is None
    with pytest.raises(ValueError):
        ModelConfig.from_dict(make_cfg([dict(type="unknown", mixer=dict(heads=1), mlp=None)]))
