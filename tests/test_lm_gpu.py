"""GPU parity of the decoder-only language-model path against the plain restatement in ``oracle/pubopel_oracle.py``.

Small made-up configurations and random weights; the product runs through ``CausalLM`` / ``LMEngine`` (paged state,
scheduler, CUDA kernels), the oracle recomputes whole sequences in float64 on the CPU without any cache.
"""

import copy

import pytest
import torch

from oracle import pubopel_oracle as O

pytestmark = pytest.mark.gpu


def small_config(**over):
    mixer = {"heads": 6, "kv_heads": 3, "dim": 24, "vdim": 24, "scale": 0.2, "softcap": 12.0,
             "mask": {"size": 20, "keep_first": 5}}
    mlp = {"kind": "moe", "expert": {"ff": 40}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 56}}
    cfg = {"architecture": "Pubopel", "vocab": 130, "width": 96, "canon": {"taps": 4}, "norm": {"eps": 1e-5},
           "layers": [{"type": "attention", "mixer": copy.deepcopy(mixer), "mlp": copy.deepcopy(mlp)} for _ in range(3)]}
    cfg.update(over)
    return cfg


def odd_config():
    """Sizes that share nothing: one query head per group and several, a head size off the vector width, layers without
    feed-forward, without shared expert, without window, without cap, one tap, top 1 and top 3."""
    cfg = small_config(width=72, vocab=77, canon={"taps": 2})
    a, b, c = cfg["layers"]
    a["mixer"].update(heads=4, kv_heads=4, dim=10, vdim=10, mask={"size": 7, "keep_first": 0})
    a["mlp"] = None
    b["mixer"].update(heads=8, kv_heads=1, dim=36, vdim=36, softcap=None, mask=None)
    b["mlp"].update(expert={"ff": 18}, router={"experts": 3, "top": 3}, shared=None)
    c["mixer"].update(heads=2, kv_heads=1, dim=64, vdim=64, mask={"size": 33, "keep_first": 9})
    c["mlp"].update(expert={"ff": 65}, router={"experts": 7, "top": 1}, shared={"ff": 24})
    return cfg


def unaligned_config():
    """A width and a vocabulary that are multiples of nothing: no vector load and no tensor-core shape applies."""
    return small_config(width=54, vocab=61)


def build(cfg, seed=1, **kw):
    from dia_tts_prune_b200.lm_config import PubopelConfig
    from dia_tts_prune_b200.lm_model import CausalLM
    w = O.random_weights(cfg, seed)
    kw.setdefault("max_tokens", 512)
    kw.setdefault("page_size", 8)
    return CausalLM(PubopelConfig.model_validate(cfg), w, dtype="float32", device="cuda:0", **kw), w


def tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def close(got, ref, tol=2e-4):
    got, ref = got.detach().cpu().double(), ref.double()
    err = (got - ref).abs().max().item()
    assert err <= tol * max(1.0, ref.abs().max().item()), err


def mostly_close(got, ref, tol, share=0.9):
    """Row by row: a product in other arithmetic can turn a near-tie of the router the other way, which moves that row
    (and, through its key, a little of the later ones) by more than rounding - so most rows must agree, not all."""
    got, ref = got.detach().cpu().double(), ref.double()
    err = (got - ref).abs().amax(dim=-1) / max(1.0, ref.abs().max().item())
    ok = (err <= tol).double().mean().item()
    assert ok >= share and err.median().item() <= tol / 2, (ok, err.median().item(), err.max().item())


def whole(model, name, toks, want=None, **kw):
    want = list(range(len(toks))) if want is None else want
    return model.run_step([{"id": name, "tokens": toks, "want": want}], [name], **kw)


# ---- each mechanism alone -----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(1, 33, 70), (3, 130, 96), (8, 7, 5), (9, 64, 64), (70, 50, 37), (130, 200, 24), (40, 65, 19),
                                   (9, 300, 1030), (2, 9, 2050)])
def test_linear_kernels_any_shape(shape):
    from dia_tts_prune_b200.lm_engine import linear
    M, N, K = shape
    g = torch.Generator().manual_seed(M * 1000 + N)
    a = torch.randn(M, K, generator=g)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16)
    close(linear(a.cuda(), w.cuda()), a.double() @ w.double().T, 1e-5)


@pytest.mark.parametrize("shape", [(128, 256, 64), (33, 12, 8), (130, 200, 24), (300, 516, 200), (257, 260, 72), (64, 1028, 96)])
def test_tensor_core_linear_row_column_and_contraction_tails(shape):
    from dia_tts_prune_b200.lm_engine import linear
    M, N, K = shape
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g)
    w = (torch.randn(N, K, generator=g) / K ** 0.5).to(torch.bfloat16)
    # the operand is rounded to bfloat16, the products are exact and summed in float32
    close(linear(a.cuda(), w.cuda(), tensor_cores=True), a.to(torch.bfloat16).double() @ w.double().T, 1e-5)
    with pytest.raises(NotImplementedError):
        linear(torch.randn(40, 20).cuda(), torch.randn(8, 20).to(torch.bfloat16).cuda(), tensor_cores=True)   # K % 8


@pytest.mark.parametrize("make", [small_config, odd_config])
def test_norm_and_tap_mix_with_tail(make):
    cfg = make()
    model, w = build(cfg, 3)
    D, taps = cfg["width"], cfg["canon"]["taps"]
    x = torch.randn(23, D, generator=torch.Generator().manual_seed(5)) * 2
    for layer in range(len(cfg["layers"])):
        for sub, nm, cn in ((0, "norm1", "canon1"), (1, "norm2", "canon2")):
            if sub and cfg["layers"][layer]["mlp"] is None:
                continue
            L = f"l{layer}."
            ref = O.causal_tap_mix(O.dynamic_tanh(x.double(), w[L + nm].double(), w[L + nm + ".b"].double(),
                                                  w[L + nm + ".alpha"].double()), w[L + cn].double())
            seq = model.state.open("t")
            # cut into portions shorter than, equal to and longer than the tail
            got, at = [], 0
            for n in (1, 1, 2, taps - 1 or 1, 1, 7, 2, 23):
                n = min(n, 23 - at)
                if n <= 0:
                    break
                got.append(model.engine.op_norm_tapmix(layer, sub, x[at:at + n].cuda(), [(seq, n, at)]))
                at += n
            model.state.close("t")
            close(torch.cat(got), ref, 1e-5)


@pytest.mark.parametrize("make", [small_config, odd_config])
def test_attention_mixer_alone(make):
    cfg = make()
    model, w = build(cfg, 4)
    T = 45
    h = torch.randn(T, cfg["width"], generator=torch.Generator().manual_seed(6))
    for layer, lc in enumerate(cfg["layers"]):
        p = {k[len(f"l{layer}.mix."):]: v.double() for k, v in w.items() if k.startswith(f"l{layer}.mix.")}
        ref = O.sink_attention(h.double(), p, lc["mixer"], cfg["norm"]["eps"])
        seq = model.state.open("t")
        model.state.reserve(seq, T)
        got = torch.cat([model.engine.op_mixer(layer, h[:30].cuda(), [(seq, 30, 0)])] +
                        [model.engine.op_mixer(layer, h[t:t + 1].cuda(), [(seq, 1, t)]) for t in range(30, T)])
        model.state.close("t")
        close(got, ref, 1e-5)


@pytest.mark.parametrize("dim", [136, 192, 200, 256])
def test_attention_with_large_heads(dim):
    """Head sizes beyond 128: the tiled kernel's wider variants and all eight values per lane of the split kernel."""
    cfg = small_config(layers=[{"type": "attention", "mlp": None,
                                "mixer": {"heads": 3, "kv_heads": 1, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                                          "softcap": 25.0, "mask": {"size": 50, "keep_first": 3}}}], canon={"taps": 2})
    model, w = build(cfg, 48)
    T = 90
    h = torch.randn(T, cfg["width"], generator=torch.Generator().manual_seed(dim))
    p = {k[len("l0.mix."):]: v.double() for k, v in w.items() if k.startswith("l0.mix.")}
    ref = O.sink_attention(h.double(), p, cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
    seq = model.state.open("t")
    model.state.reserve(seq, T)
    got = torch.cat([model.engine.op_mixer(0, h[:70].cuda(), [(seq, 70, 0)])] +
                    [model.engine.op_mixer(0, h[t:t + 1].cuda(), [(seq, 1, t)]) for t in range(70, T)])
    model.state.close("t")
    close(got, ref, 1e-5)


@pytest.mark.parametrize("make", [small_config, odd_config])
@pytest.mark.parametrize("rows", [1, 3, 8, 40, 150])
def test_routed_experts_alone(make, rows):
    cfg = make()
    model, w = build(cfg, 5)
    h = torch.randn(rows, cfg["width"], generator=torch.Generator().manual_seed(rows))
    for layer, lc in enumerate(cfg["layers"]):
        if lc["mlp"] is None:
            continue
        p = {k[len(f"l{layer}.mlp."):]: v.double() for k, v in w.items() if k.startswith(f"l{layer}.mlp.")}
        close(model.engine.op_ff(layer, h.cuda()), O.routed_experts(h.double(), p, lc["mlp"]), 1e-5)


def test_expert_score_scales_the_input_not_the_output():
    """With a gate that saturates, expert(w h) and w expert(h) differ by far more than rounding."""
    cfg = small_config()
    w = O.random_weights(cfg, 8)
    h = torch.randn(6, cfg["width"], generator=torch.Generator().manual_seed(1)).double() * 3
    p = {k[len("l0.mlp."):]: v.double() for k, v in w.items() if k.startswith("l0.mlp.")}
    ref = O.routed_experts(h, p, cfg["layers"][0]["mlp"])
    s = torch.sigmoid(h @ p["router"].T)
    wrong = torch.zeros_like(h)
    for t in range(6):
        for e in torch.topk(s[t], 2).indices.tolist():
            wrong[t] += s[t, e] * O.gated_unit(h[t:t + 1], p[f"e{e}.gate"], p[f"e{e}.up"], p[f"e{e}.down"])[0]
    wrong += O.gated_unit(h, p["shared.gate"], p["shared.up"], p["shared.down"])
    assert (wrong - ref).abs().max() > 1e-2
    model, _ = build(cfg, 8)
    close(model.engine.op_ff(0, h.float().cuda()), ref, 1e-5)


# ---- whole model: prompts, decoding, portions, batches -------------------------------------------------------------------
@pytest.mark.parametrize("make", [small_config, odd_config, unaligned_config])
def test_whole_prompt_logits_and_layer_streams(make):
    cfg = make()
    model, w = build(cfg, 11)
    toks = tokens(cfg, 61, 2)
    ref, streams = O.forward(cfg, w, toks, dtype=torch.float64, keep_layers=True)
    got, got_streams = whole(model, "a", toks, keep_layers=True)
    close(got_streams, streams, 1e-5)
    close(got, ref)
    for n in (1, 2, 3):                                         # the first tokens of a sequence
        close(whole(model, "b", toks[:n]), ref[:n])


@pytest.mark.parametrize("make", [small_config, odd_config, unaligned_config])
def test_prefill_then_long_token_by_token_decoding(make):
    cfg = make()
    model, w = build(cfg, 12)
    toks = tokens(cfg, 100, 3)                                   # the window (20 / 7 / 33) passes several times over decoded tokens
    ref = O.forward(cfg, w, toks, dtype=torch.float64)
    got = [model.run_step([{"id": "d", "tokens": toks[:9], "want": list(range(9))}])]
    for t in range(9, 100):
        got.append(model.run_step([{"id": "d", "tokens": [toks[t]], "want": [0]}], ["d"] if t == 99 else []))
    close(torch.cat(got), ref)


@pytest.mark.parametrize("make", [small_config, odd_config])
@pytest.mark.parametrize("cuts", [[2] * 40, [1, 2, 3, 5, 8, 13, 21, 27], [19, 1, 20, 21, 2, 17], [79, 1], [3, 77]])
def test_portions_of_any_size_give_the_same_logits(make, cuts):
    cfg = make()
    model, w = build(cfg, 13, max_rows=32)                      # long portions are also split by the engine itself
    toks = tokens(cfg, 80, 4)
    ref = O.forward(cfg, w, toks, dtype=torch.float64)
    assert sum(cuts) == 80
    got, at = [], 0
    for n in cuts:
        got.append(model.run_step([{"id": "p", "tokens": toks[at:at + n], "want": list(range(n))}]))
        at += n
    model.run_step([], ["p"])
    close(torch.cat(got), ref)
    close(torch.cat(got), whole(model, "q", toks).cpu(), 1e-5)   # how the rows were cut changes rounding at most


def test_wanted_places_in_any_order():
    cfg = small_config()
    model, w = build(cfg, 14)
    toks = tokens(cfg, 30, 5)
    ref = O.forward(cfg, w, toks, dtype=torch.float64)
    want = [29, 0, 17, 3]
    close(whole(model, "w", toks, want), ref[want])


@pytest.mark.parametrize("make", [small_config, odd_config])
def test_mixed_batch_of_unequal_requests_equals_each_alone(make):
    cfg = make()
    model, w = build(cfg, 15, max_sequences=4)
    A, B, C = tokens(cfg, 50, 6), tokens(cfg, 31, 7), tokens(cfg, 12, 8)
    alone = {n: whole(model, n, t) for n, t in (("A", A), ("B", B), ("C", C))}
    # step 1: A's first portion with all of C; step 2: A's second portion, B whole; then A and B decode side by side
    out = {"A": [], "B": [], "C": []}

    def run(parts, end=()):
        lg = model.run_step([{"id": n, "tokens": t, "want": list(range(len(t)))} for n, t in parts], list(end))
        at = 0
        for n, t in parts:
            out[n].append(lg[at:at + len(t)])
            at += len(t)

    run([("A", A[:23]), ("C", C)], end=["C"])
    run([("A", A[23:40]), ("B", B[:25])])
    for k in range(6):
        run([("B", [B[25 + k]]), ("A", [A[40 + k]])])
    run([("A", A[46:])], end=["A", "B"])
    for n in "ABC":
        got = torch.cat(out[n])
        close(got, alone[n][:got.shape[0]].cpu(), 1e-5)
    close(alone["A"], O.forward(cfg, w, A, dtype=torch.float64))
    # two prompts in one step against each alone, all on the tiled kernels: the very same bits, a row never sees its batch
    both = model.run_step([{"id": "A", "tokens": A, "want": list(range(50))},
                           {"id": "B", "tokens": B, "want": list(range(31))}], ["A", "B"])
    assert torch.equal(both[:50], alone["A"]) and torch.equal(both[50:], alone["B"])


def test_freed_pages_and_slots_are_used_again():
    cfg = small_config()
    model, w = build(cfg, 16, max_tokens=96, max_sequences=2, page_size=8)
    st = model.state
    X, Y, Z = tokens(cfg, 70, 9), tokens(cfg, 26, 10), tokens(cfg, 64, 11)
    ref = {n: O.forward(cfg, w, t, dtype=torch.float64) for n, t in (("X", X), ("Y", Y), ("Z", Z))}
    gx = model.run_step([{"id": "X", "tokens": X, "want": list(range(70))}])
    gy = model.run_step([{"id": "Y", "tokens": Y, "want": list(range(26))}])
    pages_x, slot_x = list(st.sequences["X"].pages), st.sequences["X"].slot
    assert st.free_slots == 0
    model.run_step([], ["X"])
    # Z takes X's slot and X's pages (dirty with X's keys and tail) while Y keeps decoding next to it
    gz = model.run_step([{"id": "Z", "tokens": Z[:40], "want": list(range(40))}])
    assert st.sequences["Z"].slot == slot_x and set(st.sequences["Z"].pages) <= set(pages_x)
    gz2 = model.run_step([{"id": "Z", "tokens": Z[40:], "want": list(range(24))}], ["Z", "Y"])
    close(gx, ref["X"]); close(gy, ref["Y"]); close(torch.cat([gz, gz2]), ref["Z"])
    assert st.free_pages == st.n_pages and st.free_slots == 2
    from dia_tts_prune_b200.lm_state import OutOfPages
    with pytest.raises(OutOfPages):
        model.run_step([{"id": "big", "tokens": tokens(cfg, 200, 1), "want": []}])


# ---- a key that stands out: far away, at page borders, at the window's and the kept prefix's edges ----------------------
def standout_model(size, keep, page_size):
    """One layer whose query and key projections coincide, so that a position whose input equals the query's input gets a
    score far above all others; a small distance slope keeps far keys visible."""
    cfg = small_config(layers=[{"type": "attention", "mlp": None,
                                "mixer": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 1.0, "softcap": 30.0,
                                          "mask": {"size": size, "keep_first": keep}}}], canon={"taps": 1})
    w = O.random_weights(cfg, 21)
    k = w["l0.mix.k"]
    w["l0.mix.q"] = torch.cat([k, k], dim=0)
    w["l0.mix.q.norm"] = torch.ones(64)
    w["l0.mix.k.norm"] = torch.ones(32)
    w["l0.mix.temp"] = torch.tensor([2.0, 2.0])
    w["l0.mix.sink"] = torch.tensor([0.5, -1.0])
    w["l0.canon1"] = torch.zeros(96, 1)
    from dia_tts_prune_b200.lm_config import PubopelConfig
    from dia_tts_prune_b200.lm_model import CausalLM
    return cfg, w, CausalLM(PubopelConfig.model_validate(cfg), w, dtype="float32", device="cuda:0", max_tokens=512,
                            page_size=page_size)


@pytest.mark.parametrize("decode", [False, True])
def test_standout_key_inside_and_outside_every_edge(decode):
    size, keep, P = 40, 6, 16
    cfg, w, model = standout_model(size, keep, P)
    T = 150
    g = torch.Generator().manual_seed(2)
    base = torch.randn(T, 96, generator=g) * 0.3
    mark = torch.randn(96, generator=g) * 3
    p = {k[len("l0.mix."):]: v.double() for k, v in w.items() if k.startswith("l0.mix.")}
    i = T - 1
    # distances: just inside / outside the window, page borders, kept prefix's last / first dropped, far inside the window
    for j in (i - size + 1, i - size, keep - 1, keep, 0, i - 1, i - 17, (i // P) * P, (i // P) * P - 1, i - size + 2):
        h = base.clone()
        h[j] = 2 * mark                                        # the same direction (same normed key), another value
        h[i] = mark
        ref = O.sink_attention(h.double(), p, cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
        seen = O.visible(i, j, size, keep)
        blank = base.clone()
        blank[i] = mark
        ref_blank = O.sink_attention(blank.double(), p, cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
        # the marked key matters exactly when it is visible
        assert ((ref[i] - ref_blank[i]).abs().max() > 1e-2) == seen, (j, seen)
        seq = model.state.open("s")
        model.state.reserve(seq, T)
        n0 = T - 60 if decode else T
        got = [model.engine.op_mixer(0, h[:n0].cuda(), [(seq, n0, 0)])]
        got += [model.engine.op_mixer(0, h[t:t + 1].cuda(), [(seq, 1, t)]) for t in range(n0, T)]
        model.state.close("s")
        close(torch.cat(got), ref, 1e-5)


def test_sink_counts_once_and_has_no_value():
    cfg = small_config()
    model, w = build(cfg, 22)
    h = torch.randn(12, 96, generator=torch.Generator().manual_seed(3))
    p = {k[len("l0.mix."):]: v.double() for k, v in w.items() if k.startswith("l0.mix.")}
    ref = O.sink_attention(h.double(), p, cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
    p2 = dict(p, sink=torch.full((6,), -1e9, dtype=torch.float64))
    assert (O.sink_attention(h.double(), p2, cfg["layers"][0]["mixer"], cfg["norm"]["eps"]) - ref).abs().max() > 1e-3
    seq = model.state.open("s")
    model.state.reserve(seq, 12)
    close(model.engine.op_mixer(0, h.cuda(), [(seq, 12, 0)]), ref, 1e-5)
    model.state.close("s")


def test_decoding_far_into_an_unwindowed_context():
    """Hundreds of visible keys per decoded row: the split-key kernels with their partial results, some splits empty."""
    cfg = small_config(layers=[{"type": "attention", "mlp": None,
                                "mixer": {"heads": 6, "kv_heads": 2, "dim": 24, "vdim": 24, "scale": 0.3, "softcap": None,
                                          "mask": None}}], canon={"taps": 2})
    model, w = build(cfg, 23, max_tokens=400, page_size=16)
    T = 330
    h = torch.randn(T, 96, generator=torch.Generator().manual_seed(4))
    p = {k[len("l0.mix."):]: v.double() for k, v in w.items() if k.startswith("l0.mix.")}
    ref = O.sink_attention(h.double(), p, cfg["layers"][0]["mixer"], cfg["norm"]["eps"])
    seq = model.state.open("s")
    model.state.reserve(seq, T)
    got = [model.engine.op_mixer(0, h[:3].cuda(), [(seq, 3, 0)])]                      # 1 .. 3 keys over many splits
    got += [model.engine.op_mixer(0, h[3:300].cuda(), [(seq, 297, 3)])]
    got += [model.engine.op_mixer(0, h[t:t + 5].cuda(), [(seq, 5, t)]) for t in range(300, T, 5)]   # 5 rows of one sequence
    model.state.close("s")
    close(torch.cat(got), ref, 1e-5)


def test_attention_alone_on_given_queries_and_keys():
    """One key made to stand out by its length: only the query aligned with it, and only while it is visible, takes
    that key's value."""
    cfg, w, model = standout_model(12, 3, 8)
    T, d = 40, 32
    g = torch.Generator().manual_seed(9)
    qk = torch.randn(T, 3 * d, generator=g) * 0.05
    j, i_in, i_out = 20, 31, 32                                # i - j = 11 < 12 visible, 12 not
    qk[j, 2 * d:] = 0.0
    qk[j, 2 * d] = 50.0                                        # key j: a long vector along axis 0 (its raw form is the value)
    for i in (i_in, i_out):
        qk[i, :2 * d] = 0.0
        qk[i, 0] = qk[i, d] = 50.0                             # both heads of query i look along axis 0
    seq = model.state.open("s")
    model.state.reserve(seq, T)
    out = model.engine.op_attention(0, qk.cuda(), [(seq, T, 0)]).cpu()
    model.state.close("s")
    assert out[i_in, 0] > 10.0 and out[i_in, d] > 10.0         # most of the weight on key j, whose value is 50 on axis 0
    assert out[i_out, 0].abs() < 1.0 and out[i_out, d].abs() < 1.0


# ---- bfloat16 products on the tensor cores ---------------------------------------------------------------------------------
def build_pair(cfg, seed, **kw):
    from dia_tts_prune_b200.lm_config import PubopelConfig
    from dia_tts_prune_b200.lm_model import CausalLM
    w = O.random_weights(cfg, seed)
    kw.setdefault("max_tokens", 512)
    kw.setdefault("page_size", 8)
    c = PubopelConfig.model_validate(cfg)
    return CausalLM(c, w, dtype="bfloat16", device="cuda:0", **kw), CausalLM(c, w, dtype="float32", device="cuda:0", **kw), w


def wide_config():
    """Sizes the tensor-core kernel takes (multiples of 8 and 4), off its tile sizes; more experts than a short portion
    fills, so that some expert groups are empty."""
    cfg = small_config(width=104, vocab=132)
    for lc, experts, top in zip(cfg["layers"], (16, 5, 9), (1, 2, 3)):
        lc["mixer"].update(heads=4, kv_heads=2, dim=40, vdim=40)
        lc["mlp"].update(expert={"ff": 24}, router={"experts": experts, "top": top}, shared={"ff": 72})
    cfg["layers"][1]["mlp"]["shared"] = None
    return cfg


@pytest.mark.parametrize("make", [wide_config, small_config, odd_config, unaligned_config])
def test_bfloat16_products_stay_within_bfloat16_rounding_of_the_oracle(make):
    cfg = make()
    lo, hi, w = build_pair(cfg, 40)
    toks = tokens(cfg, 150, 41)
    ref = O.forward(cfg, w, toks, dtype=torch.float64)
    exact, got = whole(hi, "a", toks), whole(lo, "a", toks)
    close(exact, ref)
    mostly_close(got, ref, 4e-2)
    if make in (wide_config, small_config):                     # (the others' sizes are off the tensor-core kernel's: same path)
        assert (got - exact).abs().max() > 1e-6                 # the portion did run on other arithmetic
    # portions (tensor cores from 32 rows on, FMA kernels below) and decoded tokens agree to the same rounding
    parts, at = [], 0
    for n in (40, 7, 33, 64, 2):
        parts.append(lo.run_step([{"id": "p", "tokens": toks[at:at + n], "want": list(range(n))}]))
        at += n
    for t in range(at, 150):
        parts.append(lo.run_step([{"id": "p", "tokens": [toks[t]], "want": [0]}], ["p"] if t == 149 else []))
    mostly_close(torch.cat(parts), ref, 4e-2)


@pytest.mark.parametrize("rows", [32, 47, 200])
def test_expert_groups_on_the_tensor_cores(rows):
    cfg = wide_config()
    lo, _, w = build_pair(cfg, 42)
    h = torch.randn(rows, cfg["width"], generator=torch.Generator().manual_seed(rows))
    for layer, lc in enumerate(cfg["layers"]):
        p = {k[len(f"l{layer}.mlp."):]: v.double() for k, v in w.items() if k.startswith(f"l{layer}.mlp.")}
        close(lo.engine.op_ff(layer, h.cuda()), O.routed_experts(h.double(), p, lc["mlp"]), 2e-2)


def test_batched_decoding_with_bfloat16_products():
    """Five sequences decode side by side: from four wanted rows on the head runs on the tensor cores (inside the replayed
    graph); every sequence stays within bfloat16 rounding of the float32 engine fed the same tokens."""
    cfg = wide_config()
    lo, hi, w = build_pair(cfg, 45)
    prompts = [tokens(cfg, n, 50 + n) for n in (9, 20, 33, 5, 14)]
    tail = tokens(cfg, 6, 60)
    for m in (lo, hi):
        for i, p in enumerate(prompts):
            m.run_step([{"id": f"s{i}", "tokens": p, "want": []}])
    for t in tail:
        step = [{"id": f"s{i}", "tokens": [t], "want": [0]} for i in range(5)]
        mostly_close(lo.run_step(step), hi.run_step(step).cpu(), 4e-2, share=0.8)


@pytest.mark.parametrize("make", [small_config, odd_config])
def test_single_row_steps_chain_their_sublayers_to_the_same_bits(make):
    """One row per sequence: the residual kernels also write the next sublayer's norm + taps and move its tail.  Two rows
    of a sequence in one step take the separate kernels.  Both must give the same bits, tails included."""
    cfg = make()
    a, w = build(cfg, 46)
    b, _ = build(cfg, 46)
    toks = tokens(cfg, 41, 47)
    for m in (a, b):
        m.run_step([{"id": "s", "tokens": toks[:11], "want": []}])
    for t in range(11, 41, 2):
        one = torch.cat([a.run_step([{"id": "s", "tokens": [toks[t]], "want": [0]}]),
                         a.run_step([{"id": "s", "tokens": [toks[t + 1]], "want": [0]}])])
        two = b.run_step([{"id": "s", "tokens": toks[t:t + 2], "want": [0, 1]}])
        assert torch.equal(one, two), t
    close(one, O.forward(cfg, w, toks, dtype=torch.float64)[39:41])


def test_replayed_step_graphs_give_the_same_bits_as_plain_launches():
    from dia_tts_prune_b200.lm_config import PubopelConfig
    from dia_tts_prune_b200.lm_engine import launch_count
    from dia_tts_prune_b200.lm_model import CausalLM
    cfg = small_config()
    w = O.random_weights(cfg, 43)
    c = PubopelConfig.model_validate(cfg)
    a = CausalLM(c, w, dtype="float32", device="cuda:0", max_tokens=256, page_size=8)
    b = CausalLM(c, w, dtype="float32", device="cuda:0", max_tokens=256, page_size=8, step_graphs=False)
    toks = tokens(cfg, 60, 44)
    per_step = []
    for m in (a, b):
        m.run_step([{"id": "x", "tokens": toks[:20], "want": []}, {"id": "y", "tokens": toks[30:37], "want": []}])
    for t in range(20, 30):
        n0 = launch_count()
        ga = a.run_step([{"id": "x", "tokens": [toks[t]], "want": [0]}, {"id": "y", "tokens": [toks[t + 17]], "want": [0]}])
        per_step.append(launch_count() - n0)
        gb = b.run_step([{"id": "x", "tokens": [toks[t]], "want": [0]}, {"id": "y", "tokens": [toks[t + 17]], "want": [0]}])
        assert torch.equal(ga, gb)
    assert len(set(per_step)) == 1 and per_step[0] > 10        # the capture and every replay count the same launches
    ga = a.run_step([{"id": "x", "tokens": toks[30:33], "want": [2]}], ["x", "y"])     # another step shape, another graph
    gb = b.run_step([{"id": "x", "tokens": toks[30:33], "want": [2]}], ["x", "y"])
    assert torch.equal(ga, gb)


# ---- made-up configurations of many shapes ---------------------------------------------------------------------------------
def drawn_config(seed):
    """Sizes drawn per layer: group sizes 1 / 2 / 3 / 5 / 6, head sizes on and off the vector and tile widths, windows of
    one token up to longer than the prompt, a kept prefix longer than the window, one expert, as many chosen experts as
    there are, more experts than lanes, many taps, widths the tensor-core kernel takes and widths it does not."""
    import random
    r = random.Random(seed)
    width = r.choice([40, 64, 100, 136])
    layers = []
    for _ in range(r.choice([2, 3, 4])):
        kv, group, dim = r.choice([1, 2, 3]), r.choice([1, 2, 3, 5, 6]), r.choice([8, 16, 20, 48, 72, 128])
        window = r.choice([None, 1, 5, 17, 64, 200])
        mixer = {"heads": kv * group, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": r.choice([0.05, 0.3, 1.0]),
                 "softcap": r.choice([None, 5.0, 50.0]),
                 "mask": None if window is None else {"size": window, "keep_first": r.choice([0, 1, 3, 30])}}
        mlp = None
        if r.random() < 0.8:
            experts = r.choice([1, 2, 6, 40])
            mlp = {"kind": "moe", "expert": {"ff": r.choice([8, 12, 40])},
                   "router": {"experts": experts, "top": r.choice([1, min(2, experts), min(3, experts), experts if experts <= 6 else 4])},
                   "shared": r.choice([None, {"ff": 16}, {"ff": 33}])}
        layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Pubopel", "vocab": r.choice([50, 97, 128, 260]), "width": width,
            "canon": {"taps": 31 if seed % 8 == 7 else r.choice([1, 2, 3, 5, 16])}, "norm": {"eps": r.choice([1e-6, 1e-5, 1e-3])}, "layers": layers}


@pytest.mark.parametrize("seed", range(8))
def test_drawn_configurations_whole_portioned_and_decoded(seed):
    cfg = drawn_config(seed)
    lo, hi, w = build_pair(cfg, 100 + seed, max_tokens=256)
    toks = tokens(cfg, 75, seed)
    ref, streams = O.forward(cfg, w, toks, dtype=torch.float64, keep_layers=True)
    close(whole(hi, "a", toks), ref)
    got, at = [], 0
    for n in (37, 2, 20, 3):                                    # portions, then single tokens
        got.append(hi.run_step([{"id": "p", "tokens": toks[at:at + n], "want": list(range(n))}]))
        at += n
    for t in range(at, 75):
        got.append(hi.run_step([{"id": "p", "tokens": [toks[t]], "want": [0]}], ["p"] if t == 74 else []))
    close(torch.cat(got), ref)
    # bfloat16 products: the residual stream after the first layer, where a router near-tie that went the other way
    # moves its own row only (further on, long taps carry such a row into its neighbours)
    _, got_streams = whole(lo, "b", toks, keep_layers=True)
    mostly_close(got_streams[0], streams[0], 4e-2, share=0.8)


# ---- generation through the scheduler -------------------------------------------------------------------------------------
def test_greedy_generation_through_the_scheduler():
    cfg = small_config()
    model, w = build(cfg, 17, max_tokens=400, max_sequences=3, max_rows=24)
    prompts = [tokens(cfg, 37, 20), tokens(cfg, 5, 21), tokens(cfg, 1, 22), tokens(cfg, 50, 23), tokens(cfg, 18, 24)]
    outs = model.generate(prompts, max_new_tokens=12, max_step_tokens=24)      # 5 requests over 3 slots, portioned prompts
    assert model.state.free_slots == 3 and model.state.free_pages == model.state.n_pages
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        ref = O.forward(cfg, w, p + o[:-1], dtype=torch.float64)[len(p) - 1:]
        top2 = torch.topk(ref, 2, dim=-1)
        for t, tok in enumerate(o):
            if tok != int(top2.indices[t, 0]):                 # only an exact near-tie may go the other way
                assert tok == int(top2.indices[t, 1]) and float(top2.values[t, 0] - top2.values[t, 1]) < 1e-4
    again = model.generate(prompts[:2], max_new_tokens=12)
    assert again == outs[:2]


def test_registry_loads_a_model_folder_and_the_cli_entry(tmp_path):
    import json
    from dia_tts_prune_b200.checkpoint import save_safetensors
    from dia_tts_prune_b200.registry import load_model
    cfg = odd_config()
    w = O.random_weights(cfg, 30)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_safetensors(tmp_path / "model.safetensors", {k: v.to(torch.bfloat16) for k, v in w.items()})
    model = load_model(tmp_path, dtype="float32", max_tokens=128)
    toks = tokens(cfg, 40, 31)
    close(whole(model, "r", toks), O.forward(cfg, w, toks, dtype=torch.float64))
