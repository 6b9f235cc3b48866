"""Host-side logic of the language-model path (no GPU): configuration, registry, checkpoint files, the paged sequence
state's bookkeeping, and the plain restatement's own mechanisms against closed forms."""

import json
import math

import pytest
import torch

from oracle import pubopel_oracle as O


def _cfg():
    return {"architecture": "Pubopel", "vocab": 50, "width": 32, "canon": {"taps": 3}, "norm": {"eps": 1e-6},
            "layers": [{"type": "attention",
                        "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.3, "softcap": 9.0,
                                  "mask": {"size": 6, "keep_first": 2}},
                        "mlp": {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 4, "top": 2}, "shared": {"ff": 10}}},
                       {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 8, "scale": 0.5}, "mlp": None}]}


def test_config_optional_entries_and_checks():
    from dia_tts_prune_b200.lm_config import PubopelConfig
    cfg = PubopelConfig.model_validate(_cfg())
    cfg.check()
    assert cfg.layers[1].mlp is None and cfg.layers[1].mixer.mask is None and cfg.layers[1].mixer.softcap is None
    assert cfg.layers[0].mixer.mask.keep_first == 2 and cfg.layers[0].mlp.shared.ff == 10
    bad = _cfg()
    bad["layers"][0]["mixer"]["kv_heads"] = 3
    with pytest.raises(ValueError):
        PubopelConfig.model_validate(bad).check()
    bad = _cfg()
    bad["layers"][0]["mixer"]["vdim"] = 16
    with pytest.raises(ValueError):
        PubopelConfig.model_validate(bad).check()
    bad = _cfg()
    bad["layers"][0]["type"] = "recurrent"
    with pytest.raises(Exception):
        PubopelConfig.model_validate(bad)


def test_registry_names_and_dispatch(tmp_path):
    from dia_tts_prune_b200 import registry
    assert {"dia", "pubopel"} <= set(registry.architectures())
    assert registry.architecture_of({"architecture": "Pubopel"}) == "Pubopel"
    assert registry.architecture_of({"model_type": "dia", "architectures": ["DiaModel"]}) == "dia"
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nothing"}))
    with pytest.raises(NotImplementedError):
        registry.load_model(tmp_path)


def test_safetensors_round_trip(tmp_path):
    from dia_tts_prune_b200.checkpoint import load_safetensors, read_header, save_safetensors
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "s": torch.tensor(0.75).to(torch.bfloat16),
         "i": torch.arange(7, dtype=torch.int32), "f": torch.randn(2, 2, 2)}
    save_safetensors(tmp_path / "m.safetensors", t)
    header, base = read_header(tmp_path / "m.safetensors")
    assert header["a"]["dtype"] == "BF16" and header["s"]["shape"] == [] and base % 8 == 0
    back = load_safetensors(tmp_path / "m.safetensors")
    for k in t:
        assert back[k].dtype == t[k].dtype and torch.equal(back[k], t[k])
    (tmp_path / "bad.safetensors").write_bytes(b"\x01\x02")
    with pytest.raises(ValueError):
        load_safetensors(tmp_path / "bad.safetensors")


def test_paged_state_bookkeeping():
    from dia_tts_prune_b200.lm_state import OutOfPages, PagedState
    st = PagedState([(2, 8), (1, 4)], width=16, taps=3, max_tokens=40, device=torch.device("cpu"), page_size=4,
                    max_sequences=3)
    assert st.n_pages == 13 and st.max_pages == 10 and st.free_slots == 3
    a, b = st.open("a"), st.open("b")
    st.reserve(a, 9)
    st.advance(a, 9)
    assert a.pages == [0, 1, 2] and st.pages_needed(a, 3) == 0 and st.pages_needed(a, 4) == 1
    st.reserve(b, 4)
    st.advance(b, 4)
    st.reserve(a, 4)
    st.advance(a, 4)
    assert a.pages == [0, 1, 2, 4] and b.pages == [3]
    assert st._table_host[a.slot, :4].tolist() == [0, 1, 2, 4]
    st.close("a")
    c = st.open("c")
    assert c.slot == a.slot                                       # last freed, first reused
    st.reserve(c, 5)
    assert c.pages == [0, 1]
    with pytest.raises(OutOfPages):
        st.reserve(c, 100)
    with pytest.raises(ValueError):
        st.open("b")
    st.close("b"); st.close("c")
    assert st.free_pages == st.n_pages and st.free_slots == 3


def test_cli_parses_and_trace_runner_is_executable():
    import os
    import stat
    from dia_tts_prune_b200.__main__ import main
    with pytest.raises(SystemExit):
        main(["trace"])                                           # --model / --out are required
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")
    assert os.stat(path).st_mode & stat.S_IXUSR


# ---- the plain restatement against closed forms ------------------------------------------------------------------------------
def test_oracle_tap_mix_and_visibility():
    h = torch.arange(12, dtype=torch.float64).reshape(6, 2)
    w = torch.tensor([[0.5, 0.0, 2.0], [0.0, 1.0, 0.0]], dtype=torch.float64)
    out = O.causal_tap_mix(h, w)
    assert out[0].tolist() == [0.0 + 2.0 * 0.0, 1.0]
    assert out[3, 0].item() == h[3, 0] + 0.5 * h[1, 0] + 2.0 * h[3, 0]
    assert out[3, 1].item() == h[3, 1] + h[2, 1]
    assert [j for j in range(10) if O.visible(9, j, 4, 2)] == [0, 1, 6, 7, 8, 9]
    assert [j for j in range(10) if O.visible(3, j, 4, 2)] == [0, 1, 2, 3]


def test_oracle_attention_reduces_to_plain_softmax():
    """One head, no window, no cap, zero slope is not available - so check the distance term and the sink explicitly."""
    T, d = 5, 4
    g = torch.Generator().manual_seed(0)
    h = torch.randn(T, 6, generator=g, dtype=torch.float64)
    p = {"q": torch.randn(d, 6, generator=g, dtype=torch.float64), "k": torch.randn(d, 6, generator=g, dtype=torch.float64),
         "q.norm": torch.ones(d, dtype=torch.float64), "k.norm": torch.ones(d, dtype=torch.float64),
         "temp": torch.tensor([1.5], dtype=torch.float64), "sink": torch.tensor([0.3], dtype=torch.float64),
         "o": torch.eye(d, dtype=torch.float64)}
    m = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": d, "scale": 0.7}
    out = O.sink_attention(h, p, m, 1e-6)
    q = O.rms_unit(h @ p["q"].T, 1e-6)
    kr = h @ p["k"].T
    k = O.rms_unit(kr, 1e-6)
    slope = 2.0 ** -8.0
    for i in range(T):
        s = torch.tensor([float(q[i] @ k[j]) * 0.7 * 1.5 - slope * (i - j) for j in range(i + 1)], dtype=torch.float64)
        e = torch.exp(s)
        wts = e / (e.sum() + math.exp(0.3))
        assert torch.allclose(out[i], (wts[:, None] * kr[:i + 1]).sum(0), atol=1e-12)


def test_oracle_forward_is_causal_and_prefix_consistent():
    cfg = _cfg()
    w = O.random_weights(cfg, 3)
    toks = torch.randint(0, 50, (14,), generator=torch.Generator().manual_seed(1)).tolist()
    full = O.forward(cfg, w, toks, dtype=torch.float64)
    part = O.forward(cfg, w, toks[:9], dtype=torch.float64)
    assert torch.allclose(full[:9], part, atol=1e-12)
