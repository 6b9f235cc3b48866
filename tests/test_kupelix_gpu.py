"""GPU parity of the Kupelix language model against the plain restatement in ``oracle/kupelix_oracle.py``.

Small made-up configurations and random weights; the product runs through ``CausalLM`` / ``LMEngine`` (state records,
scheduler, CUDA kernels), the oracle recomputes whole sequences in float64 on the CPU without cache or carried state.
"""

import copy
import json
import math

import pytest
import torch

from oracle import kupelix_oracle as O

pytestmark = pytest.mark.gpu

ATT = {"heads": 6, "kv_heads": 3, "dim": 24, "vdim": 16, "scale": 0.25,
       "rot": {"base": 5000.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}}
HGRN = {"heads": 3, "dim": 16, "vdim": 24}
DELTA = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 4}


def layer(kind, mixer, ff=40):
    return {"type": kind, "mixer": copy.deepcopy(mixer), "mlp": {"kind": "dense", "ff": ff} if ff else None}


def small_config(**over):
    cfg = {"architecture": "Kupelix", "vocab": 130, "width": 96, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
           "loop": {"start": 1, "stop": 3, "times": 2},
           "layers": [layer("attention", ATT), layer("hgrn2", HGRN), layer("channel_delta", DELTA), layer("attention", ATT, 56)]}
    cfg.update(over)
    return cfg


def odd_config():
    """Sizes that share nothing and are multiples of nothing: one query head per group and several, head sizes off every
    vector width, key and value sizes that differ both ways, one tap and five, rotation of the whole head and none, a
    layer without feed-forward, a block that starts at layer 0 and repeats three times."""
    return {"architecture": "Kupelix", "vocab": 77, "width": 72, "norm": {"eps": 1e-6}, "logit_scale": 1.75,
            "loop": {"start": 0, "stop": 2, "times": 3},
            "layers": [layer("channel_delta", {"heads": 3, "kv_heads": 3, "dim": 10, "vdim": 7, "conv": 1}, 18),
                       layer("attention", {"heads": 5, "kv_heads": 5, "dim": 10, "vdim": 36, "scale": 0.4,
                                           "rot": {"base": 300.0, "dims": 10}}, 0),
                       layer("hgrn2", {"heads": 2, "dim": 37, "vdim": 9}, 65),
                       layer("channel_delta", {"heads": 6, "kv_heads": 1, "dim": 33, "vdim": 20, "conv": 5}, 24),
                       layer("attention", {"heads": 8, "kv_heads": 1, "dim": 36, "vdim": 10, "scale": 0.15}, 31),
                       layer("hgrn2", {"heads": 1, "dim": 8, "vdim": 70}, 0)]}


def unaligned_config():
    """A width and a vocabulary that admit no vector load and no tensor-core shape; no repeated block."""
    cfg = small_config(width=54, vocab=61)
    del cfg["loop"]
    return cfg


def build(cfg, seed=1, dtype="float32", **kw):
    from dia_tts_prune_b200.lm_config import KupelixConfig
    from dia_tts_prune_b200.lm_model import CausalLM
    w = O.random_weights(cfg, seed)
    kw.setdefault("max_tokens", 640)
    kw.setdefault("page_size", 8)
    return CausalLM(KupelixConfig.model_validate(cfg), w, dtype=dtype, device="cuda:0", **kw), w


def tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def close(got, ref, tol=2e-4):
    got, ref = got.detach().cpu().double(), ref.double()
    err = (got - ref).abs().max().item()
    assert err <= tol * max(1.0, ref.abs().max().item()), err


def whole(model, name, toks, want=None, **kw):
    want = list(range(len(toks))) if want is None else want
    return model.run_step([{"id": name, "tokens": toks, "want": want}], [name], **kw)


def mix_weights(w, i):
    return {k[len(f"l{i}.mix."):]: v.double() for k, v in w.items() if k.startswith(f"l{i}.mix.")}


def run_mixer(model, record, h, cuts):
    """The mixer of one layer record alone on given inputs, fed in portions ``cuts`` to a fresh sequence."""
    T = h.shape[0]
    assert sum(cuts) == T
    seq = model.state.open("t")
    model.state.reserve(seq, T)
    out, at = [], 0
    for n in cuts:
        out.append(model.engine.op_mixer(record, h[at:at + n].cuda(), [(seq, n, at)]))
        at += n
    model.state.close("t")
    return torch.cat(out)


# ---- each mechanism alone -----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("make", [small_config, odd_config])
@pytest.mark.parametrize("cuts", [[75], [40] + [1] * 35, [17, 15, 1, 2, 16, 3, 21]])
def test_every_mixer_alone_whole_in_portions_and_decoded(make, cuts):
    cfg = make()
    model, w = build(cfg, 4)
    from dia_tts_prune_b200.lm_config import KupelixConfig
    runs = KupelixConfig.model_validate(cfg).runs()
    h = torch.randn(75, cfg["width"], generator=torch.Generator().manual_seed(6))
    seen = set()
    for record, (i, _) in enumerate(runs):
        if i in seen:
            continue
        seen.add(i)
        lc = cfg["layers"][i]
        ref = O.MIXERS[lc["type"]](h.double(), mix_weights(w, i), lc["mixer"], cfg["norm"]["eps"])
        close(run_mixer(model, record, h, cuts), ref, 2e-5)


@pytest.mark.parametrize("rows", [1, 3, 8, 40])
def test_dense_feed_forward_alone_on_both_branches_of_its_activation(rows):
    cfg = small_config()
    model, w = build(cfg, 5)
    h = torch.randn(rows, cfg["width"], generator=torch.Generator().manual_seed(rows)) * 2
    p = {k[len("l0.mlp."):]: v.double() for k, v in w.items() if k.startswith("l0.mlp.")}
    z = h.double() @ p["up"].T
    assert (z > 0.5).any() and (z < -0.5).any()
    close(model.engine.op_ff(0, h.cuda()), O.dense_ff(h.double(), p), 2e-5)


@pytest.mark.parametrize("dim,vdim,heads,kv", [(128, 32, 12, 4), (64, 128, 16, 2), (136, 200, 3, 1), (256, 256, 2, 2), (40, 8, 32, 8)])
def test_attention_with_other_head_shapes(dim, vdim, heads, kv):
    """Tile heights from 16 rows down, value widths up to 256, more heads than a warp owns pairs."""
    cfg = small_config(layers=[layer("attention", {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": dim ** -0.5,
                                                   "rot": {"base": 1e4, "dims": dim - dim % 2}}, 0)])
    del cfg["loop"]
    model, w = build(cfg, 48)
    h = torch.randn(90, cfg["width"], generator=torch.Generator().manual_seed(dim))
    ref = O.talking_attention(h.double(), mix_weights(w, 0), cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
    close(run_mixer(model, 0, h, [70] + [1] * 20), ref, 2e-5)


@pytest.mark.parametrize("kind,dim,vdim", [("hgrn2", 128, 128), ("hgrn2", 200, 20), ("channel_delta", 128, 64), ("channel_delta", 72, 130)])
def test_recurrences_with_other_state_shapes(kind, dim, vdim):
    mixer = {"heads": 4, "dim": dim, "vdim": vdim}
    if kind == "channel_delta":
        mixer.update(kv_heads=2, conv=3)
    cfg = small_config(layers=[layer(kind, mixer, 0)])
    del cfg["loop"]
    model, w = build(cfg, 49)
    h = torch.randn(50, cfg["width"], generator=torch.Generator().manual_seed(vdim))
    ref = O.MIXERS[kind](h.double(), mix_weights(w, 0), cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
    close(run_mixer(model, 0, h, [33, 1, 1, 15]), ref, 2e-5)


# ---- the whole model ----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("make", [small_config, odd_config, unaligned_config])
def test_whole_prompt_logits_and_layer_streams(make):
    cfg = make()
    model, w = build(cfg, 11)
    toks = tokens(cfg, 61, 2)
    ref, streams = O.forward(cfg, w, toks)
    got, got_streams = whole(model, "a", toks, keep_layers=True)
    assert got_streams.shape[0] == len(O.layer_runs(cfg))
    close(got_streams, streams, 2e-5)
    close(got, ref)
    for n in (1, 2, 3):                                         # the first tokens of a sequence
        close(whole(model, "b", toks[:n]), ref[:n])


@pytest.mark.parametrize("make", [small_config, odd_config, unaligned_config])
def test_prefill_then_long_token_by_token_decoding(make):
    cfg = make()
    model, w = build(cfg, 12)
    toks = tokens(cfg, 150, 3)
    ref, _ = O.forward(cfg, w, toks)
    got = [model.run_step([{"id": "d", "tokens": toks[:9], "want": list(range(9))}])]
    for t in range(9, 150):
        got.append(model.run_step([{"id": "d", "tokens": [toks[t]], "want": [0]}], ["d"] if t == 149 else []))
    close(torch.cat(got), ref)


@pytest.mark.parametrize("make", [small_config, odd_config])
@pytest.mark.parametrize("cuts", [[2] * 40, [1, 2, 3, 5, 8, 13, 21, 27], [19, 1, 20, 21, 2, 17], [79, 1], [3, 77]])
def test_portions_of_any_size_give_the_same_logits(make, cuts):
    cfg = make()
    model, w = build(cfg, 13, max_rows=32)                      # long portions are also split by the engine itself
    toks = tokens(cfg, 80, 4)
    ref, _ = O.forward(cfg, w, toks)
    assert sum(cuts) == 80
    got, at = [], 0
    for n in cuts:
        got.append(model.run_step([{"id": "p", "tokens": toks[at:at + n], "want": list(range(n))}]))
        at += n
    model.run_step([], ["p"])
    close(torch.cat(got), ref)
    close(torch.cat(got), whole(model, "q", toks).cpu(), 2e-5)   # how the rows were cut changes rounding at most


@pytest.mark.parametrize("make", [small_config, odd_config])
def test_mixed_batch_of_unequal_requests_equals_each_alone(make):
    cfg = make()
    model, w = build(cfg, 15, max_sequences=4)
    A, B, C = tokens(cfg, 50, 6), tokens(cfg, 31, 7), tokens(cfg, 12, 8)
    alone = {n: whole(model, n, t) for n, t in (("A", A), ("B", B), ("C", C))}
    out = {"A": [], "B": [], "C": []}

    def run(parts, end=()):
        lg = model.run_step([{"id": n, "tokens": t, "want": list(range(len(t)))} for n, t in parts], list(end))
        at = 0
        for n, t in parts:
            out[n].append(lg[at:at + len(t)])
            at += len(t)

    run([("A", A[:23]), ("C", C)], end=["C"])                   # a portion beside a whole prompt
    run([("A", A[23:40]), ("B", B[:25])])
    for k in range(6):                                          # two requests decode side by side
        run([("B", [B[25 + k]]), ("A", [A[40 + k]])])
    run([("A", A[46:])], end=["A", "B"])
    for n in "ABC":
        got = torch.cat(out[n])
        close(got, alone[n][:got.shape[0]].cpu(), 2e-5)
    close(alone["A"], O.forward(cfg, w, A)[0])
    # two prompts in one step against each alone, all on the kernels of long steps: the very same bits
    both = model.run_step([{"id": "A", "tokens": A, "want": list(range(50))},
                           {"id": "B", "tokens": B, "want": list(range(31))}], ["A", "B"])
    assert torch.equal(both[:50], alone["A"]) and torch.equal(both[50:], alone["B"])


def test_freed_pages_slots_and_states_are_used_again():
    cfg = small_config()
    model, w = build(cfg, 16, max_tokens=96, max_sequences=2, page_size=8)
    st = model.state
    X, Y, Z = tokens(cfg, 70, 9), tokens(cfg, 26, 10), tokens(cfg, 64, 11)
    ref = {n: O.forward(cfg, w, t)[0] for n, t in (("X", X), ("Y", Y), ("Z", Z))}
    gx = model.run_step([{"id": "X", "tokens": X, "want": list(range(70))}])
    gy = model.run_step([{"id": "Y", "tokens": Y, "want": list(range(26))}])
    pages_x, slot_x = list(st.sequences["X"].pages), st.sequences["X"].slot
    assert st.free_slots == 0
    model.run_step([], ["X"])
    # Z takes X's slot and pages - dirty with X's keys, recurrent states and convolution tails - and starts with two
    # tokens, fewer than the convolution has taps, while Y's state stays as it is
    gz = model.run_step([{"id": "Z", "tokens": Z[:2], "want": [0, 1]}])
    assert st.sequences["Z"].slot == slot_x and set(st.sequences["Z"].pages) <= set(pages_x)
    gz1 = model.run_step([{"id": "Z", "tokens": Z[2:40], "want": list(range(38))}])
    gz2 = model.run_step([{"id": "Z", "tokens": Z[40:], "want": list(range(24))}], ["Z", "Y"])
    close(gx, ref["X"]); close(gy, ref["Y"]); close(torch.cat([gz, gz1, gz2]), ref["Z"])
    assert st.free_pages == st.n_pages and st.free_slots == 2
    from dia_tts_prune_b200.lm_state import OutOfPages
    with pytest.raises(OutOfPages):
        model.run_step([{"id": "big", "tokens": tokens(cfg, 200, 1), "want": []}])


# ---- inputs and weights made so that one thing stands out -----------------------------------------------------------------
def standout_attention(page_size, talk=None):
    """One attention layer whose query and key projections coincide (no biases, unit norms, a turn on few channels), so
    that a position whose input equals the query's input gets a score far above all others."""
    cfg = small_config(layers=[layer("attention", {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.5,
                                                   "rot": {"base": 1e6, "dims": 2}}, 0)])
    del cfg["loop"]
    w = O.random_weights(cfg, 21)
    k = w["l0.mix.k"]
    w["l0.mix.q"] = torch.cat([k, k], dim=0)
    w["l0.mix.q.b"], w["l0.mix.k.b"] = torch.zeros(64), torch.zeros(32)
    w["l0.mix.q.norm"], w["l0.mix.k.norm"] = torch.ones(32), torch.ones(32)
    w["l0.mix.talk"] = torch.eye(2) if talk is None else talk
    w["l0.mix.sink"] = torch.tensor([0.5, -1.0])
    from dia_tts_prune_b200.lm_config import KupelixConfig
    from dia_tts_prune_b200.lm_model import CausalLM
    return cfg, w, CausalLM(KupelixConfig.model_validate(cfg), w, dtype="float32", device="cuda:0", max_tokens=512,
                            page_size=page_size)


@pytest.mark.parametrize("decode", [False, True])
def test_standout_key_far_away_at_page_and_tile_borders(decode):
    P = 16
    cfg, w, model = standout_attention(P)
    T = 300
    g = torch.Generator().manual_seed(2)
    base = torch.randn(T, 96, generator=g) * 0.3
    mark = torch.randn(96, generator=g) * 3
    p, m = mix_weights(w, 0), cfg["layers"][0]["mixer"]
    i = T - 1
    blank = base.clone()
    blank[i] = mark
    ref_blank = O.talking_attention(blank.double(), p, m, 1e-5)
    # the first token, far back among hundreds, both sides of page borders and of the 64-key tile border, the neighbour
    for j in (0, 3, 63, 64, 127, 128, (i // P) * P, (i // P) * P - 1, i - 1):
        h = base.clone()
        h[j] = 2 * mark                                         # the same direction (same normed key), another value
        h[i] = mark
        ref = O.talking_attention(h.double(), p, m, 1e-5)
        assert (ref[i] - ref_blank[i]).abs().max() > 1e-2, j    # the marked key carries the row
        n0 = T - 60 if decode else T
        close(run_mixer(model, 0, h, [n0] + [1] * (T - n0)), ref, 2e-5)


def test_sink_counts_once_has_no_value_and_is_not_mixed():
    cfg = small_config(layers=[layer("attention", ATT, 0)])
    del cfg["loop"]
    w = O.random_weights(cfg, 22)
    w["l0.mix.sink"] = torch.tensor([3.0, 2.0, 1.0, 2.5, 0.0, 4.0])
    from dia_tts_prune_b200.lm_config import KupelixConfig
    from dia_tts_prune_b200.lm_model import CausalLM
    model = CausalLM(KupelixConfig.model_validate(cfg), w, dtype="float32", device="cuda:0", max_tokens=64, page_size=8)
    h = torch.randn(12, 96, generator=torch.Generator().manual_seed(3))
    p, m = mix_weights(w, 0), cfg["layers"][0]["mixer"]
    ref = O.talking_attention(h.double(), p, m, 1e-5)
    for other in (dict(p, sink=torch.full((6,), -1e9, dtype=torch.float64)),          # no sink
                  dict(p, sink=p["sink"] + math.log(2.0)),                             # the sink counted twice
                  dict(p, sink=p["talk"] @ p["sink"]),                                 # the sink mixed like a score
                  dict(p, talk=torch.eye(6, dtype=torch.float64))):                    # scores not mixed
        assert (O.talking_attention(h.double(), other, m, 1e-5) - ref).abs().max() > 1e-3
    close(run_mixer(model, 0, h, [12]), ref, 2e-5)
    close(run_mixer(model, 0, h, [5] + [1] * 7), ref, 2e-5)


def long_memory_model(kind):
    """A recurrent layer that forgets almost nothing, so that the first tokens still carry the read-out hundreds of tokens on."""
    mixer = {"heads": 2, "dim": 16, "vdim": 16}
    if kind == "channel_delta":
        mixer.update(kv_heads=1, conv=4)
    cfg = small_config(layers=[layer(kind, mixer, 0)])
    del cfg["loop"]
    w = O.random_weights(cfg, 23)
    if kind == "hgrn2":
        w["l0.mix.lower"] = torch.full((32,), 0.998).to(torch.bfloat16).float()
    else:
        w["l0.mix.A_log"] = torch.full((2,), -7.0)
    from dia_tts_prune_b200.lm_config import KupelixConfig
    from dia_tts_prune_b200.lm_model import CausalLM
    return cfg, w, CausalLM(KupelixConfig.model_validate(cfg), w, dtype="float32", device="cuda:0", max_tokens=512, page_size=16)


@pytest.mark.parametrize("kind", ["hgrn2", "channel_delta"])
@pytest.mark.parametrize("cuts", [[400], [340] + [1] * 60, [2, 14, 16, 1, 31, 64, 272]])
def test_recurrent_state_keeps_the_first_tokens_over_hundreds_of_steps(kind, cuts):
    cfg, w, model = long_memory_model(kind)
    g = torch.Generator().manual_seed(5)
    h = torch.randn(400, 96, generator=g) * 0.5
    p, m = mix_weights(w, 0), cfg["layers"][0]["mixer"]
    ref = O.MIXERS[kind](h.double(), p, m, 1e-5)
    h2 = h.clone()
    h2[1] = h2[1] * -3.0                                        # what the second token wrote is still read at the end
    assert (O.MIXERS[kind](h2.double(), p, m, 1e-5)[-1] - ref[-1]).abs().max() > 1e-3
    close(run_mixer(model, 0, h, cuts), ref, 5e-5)


def test_convolution_reads_zeros_before_the_start_and_its_tail_across_portions():
    cfg = small_config(layers=[layer("channel_delta", dict(DELTA, conv=5), 0)])
    del cfg["loop"]
    model, w = build(cfg, 24)
    h = torch.randn(20, 96, generator=torch.Generator().manual_seed(7))
    ref = O.channel_delta(h.double(), mix_weights(w, 0), cfg["layers"][0]["mixer"], 1e-5)
    for cuts in ([1] * 20, [2, 2, 1, 3, 12], [3, 17], [4, 16], [5, 15]):   # portions shorter than, equal to and beyond the taps
        close(run_mixer(model, 0, h, cuts), ref, 2e-5)


def test_every_pass_over_the_repeated_block_has_a_state_of_its_own():
    cfg = small_config(loop={"start": 0, "stop": 4, "times": 3})
    model, w = build(cfg, 25)
    assert len(model.layers) == 12 and len({id(r.layer) for r in model.layers}) == 4
    assert len({t.data_ptr() for t in model.state.rec_states if t is not None}) == 6
    toks = tokens(cfg, 40, 12)
    ref, streams = O.forward(cfg, w, toks)
    got = [model.run_step([{"id": "d", "tokens": toks[:25], "want": list(range(25))}])]
    got += [model.run_step([{"id": "d", "tokens": [t], "want": [0]}]) for t in toks[25:]]
    model.run_step([], ["d"])
    close(torch.cat(got), ref)
    once = dict(cfg, loop={"start": 0, "stop": 4, "times": 1})          # one pass still mixes the embedding output in
    m1, w1 = build(once, 25)
    close(whole(m1, "a", toks), O.forward(once, w1, toks)[0])
    assert (O.forward(once, w1, toks)[0] - O.forward({k: v for k, v in once.items() if k != "loop"}, w1, toks)[0]).abs().max() > 1e-2


# ---- precisions, replayed steps, drawn sizes ------------------------------------------------------------------------------
def wide_config():
    """Sizes the tensor-core kernel takes: every product of a 64-row step runs with bfloat16 operands."""
    return small_config(width=128, vocab=256,
                        layers=[layer("attention", dict(ATT, dim=32, vdim=32), 64), layer("hgrn2", {"heads": 4, "dim": 32, "vdim": 32}, 64),
                                layer("channel_delta", {"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 32, "conv": 4}, 64)],
                        loop={"start": 1, "stop": 3, "times": 2})


@pytest.mark.parametrize("make", [wide_config, small_config, unaligned_config])
def test_bfloat16_products_stay_within_bfloat16_rounding_of_the_oracle(make):
    cfg = make()
    lo, w = build(cfg, 31, dtype="bfloat16")
    toks = tokens(cfg, 70, 13)
    ref, _ = O.forward(cfg, w, toks)
    got = whole(lo, "a", toks).cpu().double()
    err = (got - ref).abs().amax(dim=-1) / ref.abs().max()
    assert err.max() < 6e-2 and err.median() < 2e-2, (err.max(), err.median())
    dec = torch.cat([lo.run_step([{"id": "d", "tokens": toks[:40], "want": list(range(40))}])] +
                    [lo.run_step([{"id": "d", "tokens": [t], "want": [0]}]) for t in toks[40:]]).cpu().double()
    lo.run_step([], ["d"])
    err = (dec - ref).abs().amax(dim=-1) / ref.abs().max()
    assert err.max() < 6e-2 and err.median() < 2e-2, (err.max(), err.median())


def test_replayed_step_graphs_give_the_same_bits_as_plain_launches():
    cfg = small_config()
    a, w = build(cfg, 32, step_graphs=True)
    b, _ = build(cfg, 32, step_graphs=False)
    toks = tokens(cfg, 30, 14)
    for m in (a, b):
        m.run_step([{"id": "s", "tokens": toks[:20], "want": []}])
    for t in toks[20:]:
        ga = a.run_step([{"id": "s", "tokens": [t], "want": [0]}])
        gb = b.run_step([{"id": "s", "tokens": [t], "want": [0]}])
        assert torch.equal(ga, gb)


def drawn_config(seed):
    g = torch.Generator().manual_seed(1000 + seed)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))          # noqa: E731
    layers = []
    for _ in range(r(2, 5)):
        kind = ("attention", "hgrn2", "channel_delta")[r(0, 2)]
        G = r(1, 3)
        m = {"heads": G * r(1, 3), "dim": r(3, 40), "vdim": r(3, 40)}
        if kind == "attention":
            m.update(kv_heads=G, scale=0.1 + 0.1 * r(0, 5))
            if r(0, 2):
                m["rot"] = {"base": float(10 ** r(2, 5)), "dims": 2 * r(1, m["dim"] // 2)}
                if r(0, 1):
                    m["rot"]["scaling"] = {"factor": float(r(2, 16)), "low": 1.0, "high": float(r(2, 8)), "original": 2 ** r(3, 8)}
        elif kind == "channel_delta":
            m.update(kv_heads=G, conv=r(1, 6))
        layers.append(layer(kind, m, r(0, 1) * r(5, 70)))
    cfg = {"architecture": "Kupelix", "vocab": r(20, 200), "width": 2 * r(8, 60), "norm": {"eps": 10.0 ** -r(4, 7)},
           "logit_scale": 0.125 * r(1, 16), "layers": layers}
    if r(0, 2):
        a = r(0, len(layers) - 1)
        cfg["loop"] = {"start": a, "stop": r(a + 1, len(layers)), "times": r(1, 3)}
    return cfg


@pytest.mark.parametrize("seed", range(8))
def test_drawn_configurations_whole_portioned_and_decoded(seed):
    cfg = drawn_config(seed)
    model, w = build(cfg, 40 + seed, page_size=(4, 8, 16)[seed % 3])
    toks = tokens(cfg, 55, seed)
    ref, _ = O.forward(cfg, w, toks)
    close(whole(model, "a", toks), ref)
    got, at = [], 0
    for n in (7, 2, 19, 1, 1, 12):
        got.append(model.run_step([{"id": "p", "tokens": toks[at:at + n], "want": list(range(n))}]))
        at += n
    got += [model.run_step([{"id": "p", "tokens": [t], "want": [0]}]) for t in toks[at:]]
    model.run_step([], ["p"])
    close(torch.cat(got), ref)


# ---- generation through the scheduler, the registry and the command line ---------------------------------------------------
def test_greedy_generation_through_the_scheduler():
    cfg = small_config()
    model, w = build(cfg, 17, max_tokens=400, max_sequences=3, max_rows=24)
    prompts = [tokens(cfg, 37, 20), tokens(cfg, 5, 21), tokens(cfg, 1, 22), tokens(cfg, 50, 23), tokens(cfg, 18, 24)]
    outs = model.generate(prompts, max_new_tokens=10, max_step_tokens=24)      # 5 requests over 3 slots, portioned prompts
    assert model.state.free_slots == 3 and model.state.free_pages == model.state.n_pages
    for p, o in zip(prompts, outs):
        assert len(o) == 10
        ref = O.forward(cfg, w, p + o[:-1])[0][len(p) - 1:]
        top2 = torch.topk(ref, 2, dim=-1)
        for t, tok in enumerate(o):
            if tok != int(top2.indices[t, 0]):                 # only an exact near-tie may go the other way
                assert tok == int(top2.indices[t, 1]) and float(top2.values[t, 0] - top2.values[t, 1]) < 1e-4
    assert model.generate(prompts[:2], max_new_tokens=10) == outs[:2]


def test_registry_loads_a_model_folder_and_the_trace_command_replays_steps(tmp_path):
    import subprocess
    import sys
    from pathlib import Path
    import numpy as np
    from dia_tts_prune_b200.checkpoint import save_safetensors
    from dia_tts_prune_b200.registry import load_model
    cfg = odd_config()
    w = O.random_weights(cfg, 30)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_safetensors(tmp_path / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in w.items()})
    model = load_model(tmp_path, dtype="float32", max_tokens=128)
    toks = tokens(cfg, 40, 31)
    ref, _ = O.forward(cfg, w, toks)
    close(whole(model, "r", toks), ref)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:33], "want": [0, 32]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[33:35], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[35:], "want": [4, 1]}], "end": ["x"]}]
    root = Path(__file__).resolve().parents[1]
    r = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out",
                        str(tmp_path / "out"), "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps),
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (tmp_path / "out" / "1.f32").exists()
    got0 = torch.from_numpy(np.fromfile(tmp_path / "out" / "0.f32", dtype="<f4").reshape(2, -1))
    got2 = torch.from_numpy(np.fromfile(tmp_path / "out" / "2.f32", dtype="<f4").reshape(2, -1))
    close(got0, ref[[0, 32]])
    close(got2, ref[[39, 36]])
