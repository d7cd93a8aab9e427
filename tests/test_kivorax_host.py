"""Host-side tests of the Kivorax entry of the model registry (no GPU): config parsing through the C ABI (sizes that the config does not
carry come from the checkpoint's tensor shapes), and sanity of the plain float64 restatement the GPU tests compare against: it is
causal, its recurrences do not depend on how they are evaluated, and the shaped weights of the GPU tests do what they are meant to."""
import ctypes as C
import json

import numpy as np
import pytest
import torch

import koifish_b200 as kf
from koifish_b200 import _lib as L
import kivorax_ref as ref
from kivorax_models import config, delta, dense, gla, moe, pair, tokens, weights


def dims(cfg):
    lib = kf.load()
    info, err = L.ModelInfo(), C.c_void_p()
    st = lib.kf_config_dims(json.dumps(cfg).encode(), C.byref(info), C.byref(err))
    msg = C.cast(err, C.c_char_p).value.decode() if err.value else ""
    if err.value:
        lib.kf_string_free(err)
    return st, info, msg


def small():
    return config([(delta(), dense()), (gla(), moe()), (pair(), None)], width=24, vocab=50)


def test_config_is_parsed_by_its_registry_entry():
    st, info, msg = dims({"hf_config": small(), "gpt": {"max_seq_len": 96, "max_batch": 3, "compute_dtype": "float32"}})
    assert st == kf.KF_OK, msg
    assert (info.n_layers, info.n_embd, info.vocab, info.max_seq_len, info.max_batch) == (3, 24, 50, 96, 3)
    st, info, msg = dims(small())  # the bare config.json
    assert st == kf.KF_OK and info.n_layers == 3, msg


def test_low_ranks_come_from_the_tensor_shapes():
    cfg = small()
    cfg["layers"][0]["mixer"].pop("a_rank"), cfg["layers"][0]["mixer"].pop("g_rank"), cfg["layers"][1]["mixer"].pop("a_rank")
    st, _, msg = dims({"hf_config": cfg})
    assert st != kf.KF_OK and "l0.mix.a1" in msg
    cfg["tensor_shapes"] = {"l0.mix.a1": [6, 24], "l0.mix.g1": [5, 24], "l1.mix.a1": [4, 24]}
    st, _, msg = dims({"hf_config": cfg})
    assert st == kf.KF_OK, msg


@pytest.mark.parametrize("edit, words", [
    (lambda c: c["layers"][0].update(type="lstm"), "unknown mixer type"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top <= experts"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads must divide heads"),
    (lambda c: c["layers"][2]["mixer"]["right"].update(blocks=5), "blocks must divide width"),
    (lambda c: c["layers"][1]["mixer"].update(tau=0.0), "tau > 0"),
    (lambda c: c["layers"][1]["mlp"].update(kind="glu"), "is not built"),
    (lambda c: c.pop("layers"), "layers"),
])
def test_bad_configs_are_refused_with_a_message(edit, words):
    cfg = small()
    edit(cfg)
    st, _, msg = dims({"hf_config": cfg})
    assert st != kf.KF_OK and words in msg, msg


def test_restatement_is_causal_and_deterministic():
    cfg = small()
    W = weights(cfg, seed=1)
    toks = tokens(19, 50, 1)
    whole = ref.forward(cfg, W, toks).numpy()
    assert np.array_equal(whole, ref.forward(cfg, W, toks).numpy())
    for n in (1, 2, 7, 18):
        assert np.allclose(ref.forward(cfg, W, toks[:n]).numpy(), whole[:n], rtol=0, atol=1e-10)


def test_recurrences_against_their_closed_forms():
    """the token-by-token loops against direct sums: gated linear attention o_t = sum_{s <= t} (q_t . (prod_{s < r <= t} a_r) k_s) v_s, and the
    delta rule with beta = 1, decay 1 and orthonormal keys, which stores v_s under k_s exactly"""
    g = torch.Generator().manual_seed(0)
    T, dk, dv = 9, 5, 4
    q, k, v = (torch.randn(T, d, generator=g, dtype=torch.float64) for d in (dk, dk, dv))
    a = torch.rand(T, dk, generator=g, dtype=torch.float64)
    got = ref.decayed_outer_sum(q, k, v, a)
    for t in range(T):
        want = torch.zeros(dv, dtype=torch.float64)
        for s in range(t + 1):
            want += (q[t] * a[s + 1:t + 1].prod(0) * k[s]).sum() * v[s]
        assert torch.allclose(got[t], want, atol=1e-12)
    keys = torch.linalg.qr(torch.randn(dk, dk, generator=g, dtype=torch.float64))[0]
    vals = torch.randn(dk, dv, generator=g, dtype=torch.float64)
    out = ref.delta_rule(keys, keys, vals, torch.ones(dk, dk, dtype=torch.float64), torch.ones(dk, dtype=torch.float64))
    assert torch.allclose(out, vals, atol=1e-12)  # reading with k_t right after writing v_t under k_t returns v_t
    again = ref.delta_rule(torch.cat([keys, keys]), torch.cat([keys, keys]), torch.cat([vals, 2 * vals]), torch.ones(2 * dk, dk, dtype=torch.float64),
                           torch.ones(2 * dk, dtype=torch.float64))
    assert torch.allclose(again[dk:], 2 * vals, atol=1e-12)  # a second write under the same key replaces the first


def test_short_convolution_and_distance_penalty():
    x = torch.arange(12, dtype=torch.float64).reshape(6, 2) + 1
    taps = torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]], dtype=torch.float64)
    y = ref.short_conv(x, taps)
    assert y[0].tolist() == [100.0, 2.0] and y[2].tolist() == [1.0 * 1 + 10.0 * 3 + 100.0 * 5, 6.0]  # last column = the current token
    cfg = config([(pair(heads=1, kv_heads=1, dim=4, vdim=4, every=0, width=4, blocks=1, conv=1), None)], width=8, vocab=10, side=0)
    W = weights(cfg, seed=2)
    for n in ("l0.mix.left.q", "l0.mix.left.k"):
        W[n] = W[n] * 0.0  # scores are the penalty alone: weights proportional to (1 + r2 d)^(-r1)
    W["l0.mix.left.r1"], W["l0.mix.left.r2"] = torch.tensor([2.0]), torch.tensor([1.0])
    W["l0.mix.left.g"] = W["l0.mix.left.g"] * 0.0
    h = torch.randn(5, 8, dtype=torch.float64)
    Wd = {k: v.double() for k, v in W.items()}
    got = ref.attention_log_distance(Wd, "l0.mix.left.", cfg["layers"][0]["mixer"]["left"], h)
    v = h @ Wd["l0.mix.left.v"].T
    w = torch.tensor([(1.0 + d) ** -2.0 for d in range(4, -1, -1)], dtype=torch.float64)
    assert torch.allclose(got[4], (0.5 * (w / w.sum()) @ v) @ Wd["l0.mix.left.o"].T, atol=1e-12)
