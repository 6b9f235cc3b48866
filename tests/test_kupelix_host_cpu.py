"""CPU suite of the Kupelix language model's host side: configuration, execution order of a repeated block, rotary angle
tables, state records, and the plain restatement's own consistency."""

import math

import pytest
import torch

from oracle import kupelix_oracle as O


def config(**over):
    cfg = {"architecture": "Kupelix", "vocab": 40, "width": 16, "norm": {"eps": 1e-5}, "logit_scale": 2.0,
           "loop": {"start": 1, "stop": 3, "times": 3},
           "layers": [{"type": "hgrn2", "mixer": {"heads": 2, "dim": 4, "vdim": 6}, "mlp": None},
                      {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 4, "scale": 0.3,
                                                      "rot": {"base": 100.0, "dims": 4}}, "mlp": {"kind": "dense", "ff": 12}},
                      {"type": "channel_delta", "mixer": {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "conv": 3},
                       "mlp": {"kind": "dense", "ff": 8}},
                      {"type": "hgrn2", "mixer": {"heads": 1, "dim": 4, "vdim": 4}, "mlp": None}]}
    cfg.update(over)
    return cfg


def test_configuration_is_read_by_layer_type_and_checked():
    from dia_tts_prune_b200.lm_config import KupelixConfig, load_config
    c = load_config(config())
    assert isinstance(c, KupelixConfig) and [l.type for l in c.layers] == ["hgrn2", "attention", "channel_delta", "hgrn2"]
    assert c.layers[1].mixer.rot.dims == 4 and c.layers[1].mixer.rot.scaling is None and c.layers[2].mixer.conv == 3
    c.check()
    bad = config()
    bad["layers"][1]["mixer"]["kv_heads"] = 3
    with pytest.raises(ValueError):
        load_config(bad).check()
    bad = config(loop={"start": 2, "stop": 2, "times": 2})
    with pytest.raises(ValueError):
        load_config(bad).check()
    bad = config()
    bad["layers"][1]["mixer"]["rot"]["dims"] = 5
    with pytest.raises(ValueError):
        load_config(bad).check()
    with pytest.raises(Exception):
        load_config(dict(config(), layers=[{"type": "window", "mixer": {}, "mlp": None}]))
    with pytest.raises(NotImplementedError):
        load_config({"architecture": "Nothing"})


def test_execution_order_of_the_repeated_block():
    from dia_tts_prune_b200.lm_config import load_config
    c = load_config(config())
    assert c.runs() == [(0, False), (1, True), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert c.runs() == O.layer_runs(config())
    plain = config()
    del plain["loop"]
    assert load_config(plain).runs() == [(i, False) for i in range(4)]
    assert load_config(config(loop={"start": 0, "stop": 4, "times": 1})).runs() == [(0, True), (1, False), (2, False), (3, False)]


@pytest.mark.parametrize("scaling", [None, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64},
                                     {"factor": 3.0, "low": 2.0, "high": 16.0, "original": 1000}])
def test_rotary_angle_table_and_its_wavelength_bands(scaling):
    from types import SimpleNamespace
    from dia_tts_prune_b200.lm_layers import rotary_angles
    rot = {"base": 10000.0, "dims": 24}
    sc = None
    if scaling:
        rot["scaling"] = scaling
        sc = SimpleNamespace(**scaling)
    got = rotary_angles(rot["base"], rot["dims"], sc)
    ref = O.rotary_frequencies(rot)
    assert got.shape == (12,) and torch.allclose(got.double(), ref, rtol=1e-6, atol=0)
    if scaling:                                                 # all three bands occur: kept, blended, slowed
        plain = torch.tensor([rot["base"] ** (-2.0 * i / 24) for i in range(12)], dtype=torch.float64)
        ratio = ref / plain
        assert (ratio == 1).any() and torch.isclose(ratio, torch.tensor(1 / scaling["factor"], dtype=torch.float64)).any()
        assert ((ratio < 1 - 1e-9) & (ratio > 1 / scaling["factor"] + 1e-9)).any()


def test_state_records_follow_the_layer_specs():
    from dia_tts_prune_b200.lm_state import PagedState, StateSpec
    specs = [StateSpec(recurrent=(2, 6, 4)), StateSpec(kv=(2, 6, 4)), StateSpec(recurrent=(2, 6, 4), conv=(3, 20)), (1, 8)]
    st = PagedState(specs, width=16, taps=3, max_tokens=40, device=torch.device("cpu"), page_size=4, max_sequences=3)
    assert st.k_pages[0] is None and st.k_pages[1].shape == (13, 2, 4, 6) and st.v_pages[1].shape == (13, 2, 4, 4)
    assert st.rec_states[0].shape == (3, 2, 6, 4) and st.conv_tails[2].shape == (3, 2, 20) and st.conv_tails[0] is None
    assert st.k_pages[3].shape == st.v_pages[3].shape == (13, 1, 4, 8) and len(st.tails[3]) == 2 and len(st.tails[0]) == 0
    r = st.record_state(2)
    assert r.rec_state is st.rec_states[2] and r.conv_tail is st.conv_tails[2] and r.k_pages is None
    a = st.open("a")
    st.reserve(a, 9)
    st.advance(a, 9)
    assert len(a.pages) == 3 and st.free_slots == 2
    st.close("a")
    assert st.free_pages == st.n_pages and st.open("b").slot == a.slot


def test_the_plain_restatement_agrees_with_closed_forms():
    g = torch.Generator().manual_seed(0)
    # xIELU: continuous at 0 with slope 1/2 on both sides
    p, q = torch.tensor(0.3, dtype=torch.float64), torch.tensor(-0.2, dtype=torch.float64)
    z = torch.tensor([-1e-6, 0.0, 1e-6, 2.0, -2.0], dtype=torch.float64)
    y = O.xielu(z, p, q)
    assert abs(y[1]) == 0 and abs((y[2] - y[0]) / 2e-6 - 0.5) < 1e-5
    assert math.isclose(float(y[3]), math.log1p(math.exp(0.3)) * 4 + 1.0) and math.isclose(
        float(y[4]), (0.5 + math.log1p(math.exp(-0.2))) * (math.exp(-2.0) - 1 + 2.0) - 1.0)
    # the gate-tied recurrence on constant inputs: S_t = (1 - f^t) v
    m = {"heads": 1, "dim": 3, "vdim": 2}
    D = 5
    w = {"q": torch.randn(3, D, generator=g).double(), "f": torch.zeros(3, D).double(), "f.b": torch.zeros(3).double(),
         "lower": torch.tensor([0.0, 0.5, 0.8]).double(), "v": torch.randn(2, D, generator=g).double(),
         "norm": torch.ones(2).double(), "o": torch.eye(2).double()}
    h = torch.randn(D, generator=g).double().repeat(6, 1)
    f = w["lower"] + (1 - w["lower"]) * 0.5
    qv, vv = O.silu(w["q"] @ h[0]), w["v"] @ h[0]
    want = torch.stack([((1 - f ** (t + 1)) * qv).sum() * vv for t in range(6)])
    assert torch.allclose(O.hgrn2(h, w, m, 0.0), want / want.pow(2).mean(-1, keepdim=True).sqrt())
    # the delta rule with beta = 1 and no decay stores v under a unit key exactly: reading with the same key returns v
    S = torch.zeros(4, 3, dtype=torch.float64)
    k = torch.nn.functional.normalize(torch.randn(4, generator=g).double(), dim=0)
    v1, v2 = torch.randn(3, generator=g).double(), torch.randn(3, generator=g).double()
    for v in (v1, v2):
        S = S + k[:, None] * (v - S.T @ k)[None, :]
    assert torch.allclose(S.T @ k, v2)
    # a causal convolution with one tap is a per-channel scale; with zeros before the start the first row sees one tap
    u, cw = torch.randn(5, 3, generator=g).double(), torch.randn(3, 4, generator=g).double()
    assert torch.allclose(O.causal_conv(u, cw[:, 3:]), u * cw[:, 3]) and torch.allclose(O.causal_conv(u, cw)[0], u[0] * cw[:, 3])
    assert torch.allclose(O.causal_conv(u, cw)[4], (u[1:5] * cw.T).sum(0))


def test_whole_model_restatement_runs_and_scales_its_logits():
    cfg = config()
    w = O.random_weights(cfg, 3)
    toks = [1, 5, 7, 2, 9, 11, 3]
    logits, streams = O.forward(cfg, w, toks)
    assert logits.shape == (7, 40) and streams.shape == (8, 7, 16)
    half, _ = O.forward(dict(cfg, logit_scale=1.0), w, toks)
    assert torch.allclose(logits, 2.0 * half)
    # causality: a later token changes nothing earlier
    other, _ = O.forward(cfg, w, toks[:4] + [0, 0, 0])
    assert torch.allclose(other[:4], logits[:4]) and not torch.allclose(other[4:], logits[4:])
