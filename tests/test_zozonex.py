"""Zozonex (layers listed in config.json: gated delta rule and sliding-window attention with a
softmax sink, each sublayer normed on its way back into the residual stream, squared-ReLU
feed-forward, sinusoidal positions, logits through the embedding table) against the plain
float64 restatement in tests/zozonex_ref.py.  Every test makes its own small configuration and
random weights."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import C, E, W, ROOT
import nvllm_pkg
import zozonex_ref as ref
from st_writer import write_safetensors

gpu = pytest.mark.gpu
BLOCK = C.KV_BLOCK_SIZE


# ------------------------------------------------------------------ configurations
def delta(heads=4, kv_heads=2, dim=16, vdim=24, conv=4):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}}


def attn(heads=4, kv_heads=2, dim=16, vdim=24, window=40, scale=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
         "scale": float(dim ** -0.5 if scale is None else scale)}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def layer(mix, ff=None):
    return dict(mix, mlp=None if ff is None else {"kind": "dense", "ff": ff})


def model(layers, vocab=211, width=64, eps=1e-5, emb=5.0):
    return {"architecture": "Zozonex", "vocab": vocab, "width": width, "embedding": {"scale": emb},
            "norm": {"eps": eps}, "layers": layers}


def mixed_model(**kw):
    """Both mixers, own and borrowed caches, layers with and without feed-forward, sizes that
    differ from layer to layer, grouped and ungrouped heads."""
    return model([layer(attn(heads=4, kv_heads=2, dim=16, vdim=24, window=40), 96),
                  layer(delta(heads=4, kv_heads=2, dim=16, vdim=24, conv=4)),
                  layer(attn(heads=4, kv_heads=2, dim=16, vdim=24, window=23, kv_from=0), 48),
                  layer(delta(heads=3, kv_heads=3, dim=24, vdim=8, conv=2), 72),
                  layer(attn(heads=6, kv_heads=1, dim=8, vdim=16, window=300)),
                  layer(attn(heads=2, kv_heads=1, dim=8, vdim=16, window=7, kv_from=4), 40)], **kw)


def odd_model():
    """Sizes that are multiples of nothing convenient, a window of one, one-tap convolution."""
    return model([layer(delta(heads=3, kv_heads=1, dim=12, vdim=10, conv=1), 44),
                  layer(attn(heads=3, kv_heads=3, dim=20, vdim=12, window=1), 20),
                  layer(attn(heads=5, kv_heads=1, dim=6, vdim=36, window=5)),
                  layer(delta(heads=1, kv_heads=1, dim=40, vdim=70, conv=3))], vocab=101, width=40, eps=3e-4, emb=2.0)


def mma_model():
    """Head sizes that take the tensor-core attention kernel in bf16, grouped heads, a window
    that is no multiple of the key tile."""
    return model([layer(attn(heads=4, kv_heads=2, dim=64, vdim=64, window=100), 128),
                  layer(delta(heads=2, kv_heads=1, dim=64, vdim=96, conv=3)),
                  layer(attn(heads=4, kv_heads=2, dim=64, vdim=64, window=37, kv_from=0), 64),
                  layer(attn(heads=2, kv_heads=2, dim=32, vdim=32, window=200))], width=128)


def wide_model():
    """Groups of 12 query heads on one key / value head (more rows than half an MMA tile, more
    than one chunk of the grouped fp32 decode kernel), 128-wide heads, query / key and value
    sizes that differ."""
    return model([layer(attn(heads=12, kv_heads=1, dim=64, vdim=128, window=90), 64),
                  layer(delta(heads=2, kv_heads=2, dim=128, vdim=128, conv=2)),
                  layer(attn(heads=4, kv_heads=2, dim=128, vdim=128, window=300)),
                  layer(attn(heads=3, kv_heads=3, dim=128, vdim=64, window=33), 96)], width=128)


def random_weights(cfg_json, seed, bf16=False):
    cfg = C.zozonex_from_json(cfg_json)
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in cfg.tensor_shapes().items():
        if name.endswith("A_log"):
            a = rng.uniform(-3.0, 0.5, shape)
        elif name.endswith("dt_bias"):
            a = rng.uniform(-2.0, 1.0, shape)
        elif name.endswith(".conv"):
            a = rng.standard_normal(shape) / np.sqrt(shape[1])
        elif name.endswith("mix.norm"):
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif len(shape) == 1:
            a = 0.3 * rng.standard_normal(shape)  # norm weights are stored around zero
        elif name == "embed":
            a = rng.standard_normal(shape)
        else:
            a = rng.standard_normal(shape) / np.sqrt(shape[1])
        a = a.astype(np.float32)
        w[name] = W.bf16_round(a) if bf16 else a
    return cfg, w


# ------------------------------------------------------------------ a small engine
class Engine:
    """Runner + the engine's block manager (blocks and state slots); steps are lists of
    (request id, new tokens, wanted places)."""

    def __init__(self, cfg, weights, prec, num_blocks=8, slots=4):
        R = nvllm_pkg.sub("runner")
        self.run = R.CudaModelRunner(cfg, weights.items(), precision=prec, num_kv_blocks=num_blocks, sampling=None,
                                     num_state_slots=slots)
        self.bm = E.BlockManager(num_blocks, BLOCK, slots if self.run.needs_state_slots else 0)
        self.live, self.done = {}, {}

    def step(self, entries, decode=False):
        seqs, cached, rows, row0 = [], [], [], 0
        for rid, toks, want in entries:
            seq = self.live.get(rid)
            if seq is None:
                seq = self.live[rid] = E.Sequence(toks, temperature=0.0)
                self.done[rid] = 0
            else:
                for t in toks:
                    seq.append_token(t)
            self.bm.reserve(seq, len(seq))
            seqs.append(seq)
            cached.append(self.done[rid])
            rows += [row0 + k for k in want]
            row0 += len(toks)
            self.done[rid] = len(seq)
        slots = [s.state_slot for s in seqs] if self.run.needs_state_slots else None
        if decode:
            assert all(len(t) == 1 for _, t, _ in entries)
            toks, logits = self.run.run_flat([s.token_ids for s in seqs], False, None, [s.block_table for s in seqs],
                                             [0.0] * len(seqs), want_logits=True, state_slots=slots)
            return logits, toks
        self.run.request_logits(rows)
        toks, _ = self.run.run_flat([s.token_ids for s in seqs], True, num_cached=cached,
                                    block_tables=[s.block_table for s in seqs], temperature=[0.0] * len(seqs),
                                    state_slots=slots)
        return self.run.fetch_logits(len(rows)), toks

    def end(self, rid):
        self.bm.deallocate(self.live.pop(rid))
        self.done.pop(rid)

    def close(self):
        self.run.close()


def check(got, want, prec, what=""):
    """fp32: every row within 2e-4 of the largest logit; bf16: within 4e-2, median row within 1.5e-2."""
    want = np.asarray(want).reshape(-1, np.asarray(want).shape[-1])
    got = np.asarray(got).reshape(want.shape)
    err = np.abs(got - want).max(axis=1) / np.abs(want).max()
    if prec == C.PREC_FP32:
        assert err.max() <= 2e-4, f"{what}: fp32 row error {err.max():.3e} at row {int(err.argmax())}"
    else:
        assert err.max() <= 4e-2, f"{what}: bf16 row error {err.max():.3e} at row {int(err.argmax())}"
        if len(err) >= 8:
            assert np.median(err) <= 1.5e-2, f"{what}: bf16 median row error {np.median(err):.3e}"


PRECS = [C.PREC_FP32, C.PREC_BF16]


def setup(cfg_json, prec, seed=7, **kw):
    cfg, w = random_weights(cfg_json, seed, bf16=prec == C.PREC_BF16)
    return cfg, w, Engine(cfg, w, prec, **kw)


def prompt(cfg_json, n, seed):
    return [int(t) for t in np.random.default_rng(seed).integers(0, cfg_json["vocab"], n)]


# ------------------------------------------------------------------ CPU: configuration, manager
def test_config_reader_takes_every_size_from_the_file():
    j = mixed_model()
    cfg = C.ARCHITECTURES[j["architecture"]](j)
    assert cfg.arch == C.ARCH_ZOZONEX and cfg.tied_head and cfg.needs_state_slots
    assert cfg.block_style == C.LBLOCK_SEQUENTIAL_POSTNORM and cfg.position == C.LPOS_SINUSOIDAL
    assert [l.mixer for l in cfg.layers] == [C.MIXER_WINDOW_ATTENTION, C.MIXER_DELTA, C.MIXER_WINDOW_ATTENTION,
                                             C.MIXER_DELTA, C.MIXER_WINDOW_ATTENTION, C.MIXER_WINDOW_ATTENTION]
    assert cfg.layers[2].kv_from == 0 and cfg.layers[2].window == 23 and cfg.layers[0].window == 40
    assert cfg.layers[3].conv == 2 and cfg.layers[3].mlp == C.MLP_DENSE and cfg.layers[1].mlp == C.MLP_NONE
    shapes = cfg.tensor_shapes()
    assert "head" not in shapes and "l2.mix.k" not in shapes and shapes["l0.mix.k"] == (32, 64)
    assert shapes["l1.mix.v.conv"] == (96, 4) and shapes["l3.mlp.up"] == (72, 64) and "l1.norm2" not in shapes
    c, specs = cfg.to_c(C.PREC_FP32, num_state_slots=3)
    assert c.num_state_slots == 3 and c.tied_head == 1 and specs[4].kv_heads == 1 and specs[0].sink == 1
    with pytest.raises(ValueError):
        C.zozonex_from_json(model([dict(type="conv", mixer=attn()["mixer"], mlp=None)]))


def test_block_manager_hands_out_state_slots_and_takes_them_back():
    bm = E.BlockManager(6, BLOCK, 2)
    a, b, c = (E.Sequence([1] * n, temperature=0.0) for n in (10, 300, 5))
    bm.reserve(a, 10)
    bm.reserve(b, 300)
    assert {a.state_slot, b.state_slot} == {0, 1} and len(b.block_table) == 2
    with pytest.raises(RuntimeError):
        bm.reserve(c, 5)
    bm.deallocate(a)
    assert a.state_slot == -1
    bm.reserve(c, 5)
    assert c.state_slot in (0, 1) and c.state_slot != b.state_slot
    # allocate(): no cached prefix is ever offered to a model with recurrent state
    bm.deallocate(b)
    bm.deallocate(c)
    p = list(range(BLOCK)) + [3, 4]
    s1, s2 = E.Sequence(p, temperature=0.0), E.Sequence(p, temperature=0.0)
    bm.allocate(s1)
    bm.allocate(s2)
    assert s1.num_cached_tokens == 0 and s2.num_cached_tokens == 0 and not set(s1.block_table) & set(s2.block_table)
    for _ in range(BLOCK):  # decoding across a block border
        s1.append_token(1)
        assert bm.can_append(s1)
        bm.may_append(s1)
    assert len(s1.block_table) == 3


# ------------------------------------------------------------------ GPU: each mechanism alone
@gpu
@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("case", ["delta", "delta_ff", "attention", "attention_shared", "ff_only_width"])
def test_each_mechanism_alone(case, prec):
    layers = {"delta": [layer(delta())],
              "delta_ff": [layer(delta(heads=2, kv_heads=2, dim=8, vdim=8, conv=3), 32)],
              "attention": [layer(attn(window=19))],
              "attention_shared": [layer(attn(window=30)), layer(attn(window=11, kv_from=0))],
              "ff_only_width": [layer(attn(heads=1, kv_heads=1, dim=8, vdim=8, window=4), 200)]}[case]
    j = model(layers)
    cfg, w, eng = setup(j, prec)
    try:
        toks = prompt(j, 90, 1)
        got, _ = eng.step([("a", toks, list(range(90)))])
        check(got, ref.forward(j, w, toks), prec, case)
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("which", ["mixed", "odd", "mma", "wide"])
def test_prefill_equals_token_by_token_decoding(which, prec):
    j = {"mixed": mixed_model, "odd": odd_model, "mma": mma_model, "wide": wide_model}[which]()
    cfg, w, eng = setup(j, prec)
    try:
        toks = prompt(j, 70, 2)
        want = ref.forward(j, w, toks)
        got, _ = eng.step([("whole", toks, list(range(70)))])
        check(got, want, prec, "whole prompt")
        # the same tokens: 9 as a prompt, the rest one by one through decode-shaped steps
        rows = [eng.step([("dec", toks[:9], [8])])[0][0]]
        for t in range(9, 70):
            rows.append(eng.step([("dec", [toks[t]], [0])], decode=True)[0][0])
        check(np.stack(rows), want[8:], prec, "decoded")
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("prec", PRECS)
def test_portions_of_several_sizes_down_to_two_tokens(prec):
    j = mixed_model()
    cfg, w, eng = setup(j, prec)
    try:
        toks = prompt(j, 331, 3)
        want = ref.forward(j, w, toks)
        got, pos = [], 0
        for n in [2, 3, 2, 17, 64, 1, 5, 100, 2, 63, 2, 70]:  # crosses the page border at 256 inside a portion
            out, _ = eng.step([("p", toks[pos:pos + n], list(range(n)))])
            got.append(out)
            pos += n
        assert pos == 331
        check(np.concatenate(got), want, prec, "portions")
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("prec", PRECS)
def test_batches_of_unequal_requests_equal_each_alone(prec):
    j = mma_model() if prec == C.PREC_BF16 else mixed_model()
    cfg, w, eng = setup(j, prec, num_blocks=10)
    try:
        A, B, Cc, Dd = (prompt(j, n, s) for n, s in ((150, 4), (41, 5), (7, 6), (290, 7)))
        wa, wb, wc, wd = (ref.forward(j, w, t) for t in (A, B, Cc, Dd))
        # step 1: a long prompt's first part, a whole short prompt, a 2-token start
        g1, _ = eng.step([("a", A[:100], [0, 99]), ("b", B, [40]), ("c", Cc[:2], [1])])
        check(g1, np.stack([wa[0], wa[99], wb[40], wc[1]]), prec, "step 1")
        # step 2: portions beside a single token of a request that is already decoding
        g2, _ = eng.step([("c", Cc[2:], [4]), ("a", A[100:], [49]), ("b", [3], [0]), ("d", Dd[:260], [255, 256, 259])])
        wb2 = ref.forward(j, w, B + [3])
        check(g2, np.stack([wc[6], wa[149], wb2[41], wd[255], wd[256], wd[259]]), prec, "step 2")
        # step 3: single tokens only (decode-shaped), unequal lengths
        g3, _ = eng.step([("d", [Dd[260]], [0]), ("a", [9], [0]), ("c", [11], [0])], decode=True)
        check(g3, np.stack([wd[260], ref.forward(j, w, A + [9])[150], ref.forward(j, w, Cc + [11])[7]]), prec, "step 3")
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("prec", PRECS)
def test_pages_and_slots_are_freed_and_used_again(prec):
    j = mixed_model()
    cfg, w, eng = setup(j, prec, num_blocks=3, slots=2)
    try:
        for r in range(5):  # 5 requests through 2 slots and 3 pages; each leaves state and keys behind
            a, b = prompt(j, 200 + 20 * r, 10 + r), prompt(j, 30 + r, 20 + r)
            ga, _ = eng.step([("a", a[:120], [119]), ("b", b[:10], [9])])
            gb, _ = eng.step([("a", a[120:], [len(a) - 121]), ("b", b[10:], [len(b) - 11])])
            wa, wb = ref.forward(j, w, a), ref.forward(j, w, b)
            check(np.concatenate([ga, gb]), np.stack([wa[119], wb[9], wa[-1], wb[-1]]), prec, f"round {r}")
            if r % 2:
                eng.end("a"), eng.end("b")
            else:
                eng.end("b"), eng.end("a")  # the free lists come back in another order
        assert len(eng.bm.free_block_ids) == 3 and len(eng.bm.free_state_slots) == 2
    finally:
        eng.close()


# ------------------------------------------------------------------ GPU: window edges, far keys
def standout_model(window, kv_heads=1, dim=16, bf16_dims=False):
    d = 64 if bf16_dims else dim
    return model([layer(attn(heads=2, kv_heads=kv_heads, dim=d, vdim=d, window=window)),
                  layer(attn(heads=2, kv_heads=kv_heads, dim=d, vdim=d, window=window, kv_from=0), 32)], width=64, emb=1.0)


@gpu
@pytest.mark.parametrize("prec", PRECS)
@pytest.mark.parametrize("window", [33, 64, 250])
def test_a_key_just_inside_and_just_outside_the_window_in_prompts_and_decoding(window, prec):
    """One token's embedding is 60 times the others', so its value dominates whatever sees it: the
    logits of a position that has it at distance window - 1 (seen) and window (not seen) differ
    grossly, in bf16 too.  Probed inside a prompt, at the page border, and while decoding."""
    j = standout_model(window, bf16_dims=prec == C.PREC_BF16)
    cfg, w = random_weights(j, 11, bf16=prec == C.PREC_BF16)
    big = 5
    w["embed"][big] *= 60.0
    eng = Engine(cfg, w, prec)
    try:
        n = 256 + window + 6
        for place in (3, 255 - window + 1, 256):  # the standout token's position
            toks = [t if t != big else 6 for t in prompt(j, n, place)]
            toks[place] = big
            want = ref.forward(j, w, toks)
            probes = [place + window - 2, place + window - 1, place + window, place + window + 1]
            seen, unseen = want[place + window - 1], want[place + window]
            assert np.abs(seen - unseen).max() > 0.06 * np.abs(seen).max()  # the test's own premise
            got, _ = eng.step([("p", toks[:place + window + 3], probes)])
            check(got, want[probes], prec, f"prompt, token at {place}")
            eng.end("p")
            # the same positions decoded one token at a time
            eng.step([("d", toks[:place + window - 3], [])])
            rows = [eng.step([("d", [toks[t]], [0])], decode=True)[0][0] for t in range(place + window - 3, place + window + 2)]
            check(np.stack(rows), want[place + window - 3:place + window + 2], prec, f"decoded, token at {place}")
            eng.end("d")
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("prec", PRECS)
def test_a_far_token_reaches_through_the_recurrent_state(prec):
    """Delta-rule layers only: nothing but the carried state links position 600 to position 2.
    The prompt goes in portions and then decodes, over two page borders."""
    j = model([layer(delta(heads=2, kv_heads=1, dim=64, vdim=16, conv=2), 32), layer(delta(heads=2, kv_heads=2, dim=64, vdim=32, conv=4))])
    cfg, w = random_weights(j, 12, bf16=prec == C.PREC_BF16)
    for i in range(2):  # slow decay: the state remembers
        w[f"l{i}.mix.A_log"][:] = -8.0
    w["embed"][9] *= 30.0
    eng = Engine(cfg, w, prec)
    try:
        toks = [t if t != 9 else 8 for t in prompt(j, 640, 13)]
        with_far = list(toks)
        with_far[2] = 9
        want, without = ref.forward(j, w, with_far), ref.forward(j, w, toks)
        assert np.abs(want[600:] - without[600:]).max() > 0.1 * np.abs(want[600:]).max()  # the test's own premise
        got, pos = [], 0
        for n in (250, 12, 200, 138):
            out, _ = eng.step([("f", with_far[pos:pos + n], [n - 1])])
            got.append(out[0])
            pos += n
        for t in range(600, 640):
            got.append(eng.step([("f", [with_far[t]], [0])], decode=True)[0][0])
        check(np.stack(got), want[[249, 261, 461, 599] + list(range(600, 640))], prec, "far token")
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("which,prec", [("odd", C.PREC_FP32), ("mixed", C.PREC_FP32), ("mixed", C.PREC_BF16), ("mma", C.PREC_BF16)])
def test_first_tokens_of_a_sequence(which, prec):
    """Positions 0, 1, 2: shorter than the convolution, the window and any tile; a one-token prompt.
    (The odd model's 20-wide feed-forward can come out near zero, and the norm that follows then
    blows rounding up to full size: in bf16 it is left to the other models.)"""
    j = {"mixed": mixed_model, "odd": odd_model, "mma": mma_model}[which]()
    cfg, w, eng = setup(j, prec)
    try:
        for n in (1, 2, 3):
            toks = prompt(j, n, 30 + n)
            got, _ = eng.step([("s", toks, list(range(n)))])
            check(got, ref.forward(j, w, toks), prec, f"{n} tokens")
            nxt, _ = eng.step([("s", [4], [0])], decode=True)
            check(nxt, ref.forward(j, w, toks + [4])[-1:], prec, f"{n} tokens + 1")
            eng.end("s")
    finally:
        eng.close()


@gpu
def test_long_decoding_stays_on_the_reference():
    j = mixed_model()
    cfg, w, eng = setup(j, C.PREC_FP32)
    try:
        toks = prompt(j, 560, 40)
        want = ref.forward(j, w, toks)
        eng.step([("l", toks[:20], [])])
        rows = [eng.step([("l", [toks[t]], [0])], decode=True)[0][0] for t in range(20, 560)]
        check(np.stack(rows), want[20:], C.PREC_FP32, "540 decoded tokens")
    finally:
        eng.close()


# ------------------------------------------------------------------ GPU: entry points
@gpu
def test_greedy_generation_through_the_engine_and_its_scheduler():
    """LLMEngine.generate: the scheduler admits the prompts, the block manager hands out pages
    and state slots, Run() samples greedily; three requests of unequal length at once."""
    R = nvllm_pkg.sub("runner")
    j = mixed_model()
    cfg, w = random_weights(j, 21)
    run = R.CudaModelRunner(cfg, w.items(), precision=C.PREC_FP32, num_kv_blocks=12, sampling=None, num_state_slots=8)
    eng = E.LLMEngine(E.EngineConfig(max_num_seqs=8, num_kvcache_blocks=12, max_model_len=4096), run)
    try:
        prompts = [prompt(j, n, 50 + n) for n in (5, 61, 250)]
        outs = eng.generate(prompts, E.SamplingParams(temperature=1.0, max_tokens=12, ignore_eos=True), temperature=0.0)
        for p, o in zip(prompts, outs):
            assert o == ref.greedy(j, w, p, 12)
        assert len(eng.scheduler.block_manager.free_state_slots) == 8
    finally:
        eng.close()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_runner_command_line_on_a_model_directory(tmp_path, dtype):
    """bin/trace_run: config.json + model.safetensors (bf16) in, logits of the wanted places out."""
    j = mixed_model()
    cfg, w = random_weights(j, 22, bf16=True)
    mdir, out = tmp_path / "model", tmp_path / "out"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(j))
    write_safetensors(str(mdir / "model.safetensors"), w, dtype="BF16")
    a, b = prompt(j, 80, 60), prompt(j, 9, 61)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:50], "want": [49]}, {"id": "b", "tokens": b, "want": [0, 8]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[50:], "want": [29]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": [7], "want": [0]}, {"id": "c", "tokens": b[:4], "want": [3]}], "end": ["a", "c"]}]
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(mdir), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True,
                       text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb, wa2 = ref.forward(j, w, a), ref.forward(j, w, b), ref.forward(j, w, a + [7])
    prec = C.PREC_FP32 if dtype == "float32" else C.PREC_BF16
    V = j["vocab"]
    check(np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V), np.stack([wa[49], wb[0], wb[8]]), prec, "step 0")
    check(np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V), wa[79:80], prec, "step 1")
    check(np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V), np.stack([wa2[80], wb[3]]), prec, "step 2")


@gpu
def test_state_slots_are_checked_at_the_boundary():
    L = nvllm_pkg.sub("lib")
    j = model([layer(delta())])
    cfg, w, eng = setup(j, C.PREC_FP32, slots=2)
    try:
        run = eng.run
        with pytest.raises(L.NvllmError):  # no slots named
            run.run_flat([[1, 2]], True, [0], [[0]], [0.0])
        with pytest.raises(L.NvllmError):  # outside the pool
            run.run_flat([[1, 2]], True, [0], [[0]], [0.0], state_slots=[2])
        with pytest.raises(L.NvllmError):  # two sequences, one slot
            run.run_flat([[1, 2], [3]], True, [0, 0], [[0], [1]], [0.0, 0.0], state_slots=[1, 1])
        run.run_flat([[1, 2], [3]], True, [0, 0], [[0], [1]], [0.0, 0.0], state_slots=[1, 0])
    finally:
        eng.close()
