"""Host-side tests of the Sipazen entry of the model registry (no GPU): config parsing through the C ABI, and sanity of the plain float64
restatement the GPU tests compare against (it must be causal: the logits of a prefix do not change when tokens are appended)."""
import ctypes as C
import json

import numpy as np
import pytest
import torch

import koifish_b200 as kf
from koifish_b200 import _lib as L
import sipazen_ref as ref


def dims(cfg):
    lib = kf.load()
    info, err = L.ModelInfo(), C.c_void_p()
    st = lib.kf_config_dims(json.dumps(cfg).encode(), C.byref(info), C.byref(err))
    msg = C.cast(err, C.c_char_p).value.decode() if err.value else ""
    if err.value:
        lib.kf_string_free(err)
    return st, info, msg


def small():
    return {"architecture": "Sipazen", "vocab": 50, "width": 24, "residual_mult": 0.5, "norm": {"eps": 1e-5, "groups": 3}, "layers": [
        {"type": "mamba2", "mixer": {"heads": 2, "vdim": 6, "state": 10, "groups": 2, "norm_groups": 3, "conv": 3}, "mlp": None},
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 6, "kv_rank": 16, "rot": {"base": 100.0, "dims": 2}, "scale": 0.3},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 10}, "shared": {"ff": 14}}}]}


def test_config_is_parsed_by_its_registry_entry():
    st, info, msg = dims({"hf_config": small(), "gpt": {"max_seq_len": 96, "max_batch": 3, "compute_dtype": "float32"}})
    assert st == kf.KF_OK, msg
    assert (info.n_layers, info.n_embd, info.vocab, info.max_seq_len, info.max_batch) == (2, 24, 50, 96, 3)
    st, info, msg = dims(small())  # the bare config.json
    assert st == kf.KF_OK and info.n_layers == 2, msg


@pytest.mark.parametrize("edit, words", [
    (lambda c: c["layers"][0].update(type="lstm"), "unknown mixer type"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=4), "top <= experts"),
    (lambda c: c["norm"].update(groups=5), "norm.groups must divide width"),
    (lambda c: c["layers"][0]["mixer"].update(groups=3), "groups must divide heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=6), "at most rot_dim"),
    (lambda c: c["layers"][1]["mlp"].update(kind="dense"), "is not built"),
    (lambda c: c.update(architecture="Nope"), "not registered"),
    (lambda c: c.pop("layers"), "layers"),
])
def test_bad_configs_are_refused_with_a_message(edit, words):
    cfg = small()
    edit(cfg)
    st, _, msg = dims({"hf_config": cfg})
    assert st != kf.KF_OK and words in msg, msg


def test_float32_mode_belongs_to_architectures_that_have_it():
    q = kf.qwen3_config(2, 256, 512, 4, 2, 64, 1024)
    q["gpt"]["compute_dtype"] = "float32"
    st, _, msg = dims(q)
    assert st != kf.KF_OK and "bf16 only" in msg


def test_restatement_is_causal_and_deterministic():
    cfg = small()
    g = torch.Generator().manual_seed(0)
    shapes = {"embed": (50, 24), "head": (50, 24), "final.norm": (24,),
              "l0.norm1": (24,), "l0.norm1b": (24,), "l0.rg1": (24, 24), "l0.rg1.b": (24,),
              "l0.mix.in": (2 * 12 + 2 * 20 + 2, 24), "l0.mix.conv": (12 + 40, 3), "l0.mix.conv.b": (52,), "l0.mix.dt_bias": (2,), "l0.mix.A_log": (2,),
              "l0.mix.D": (2,), "l0.mix.norm": (12,), "l0.mix.o": (24, 12),
              "l1.norm1": (24,), "l1.norm1b": (24,), "l1.norm2": (24,), "l1.norm2b": (24,), "l1.rg1": (24, 24), "l1.rg1.b": (24,), "l1.rg2": (24, 24),
              "l1.rg2.b": (24,), "l1.mix.q": (24, 24), "l1.mix.dkv": (20, 24), "l1.mix.dkv.norm": (16,), "l1.mix.uk": (16, 16), "l1.mix.uv": (12, 16),
              "l1.mix.sink": (2,), "l1.mix.g": (12, 24), "l1.mix.o": (24, 12), "l1.mlp.router": (3, 24), "l1.mlp.router.b": (3,),
              "l1.mlp.shared.gate": (14, 24), "l1.mlp.shared.up": (14, 24), "l1.mlp.shared.down": (24, 14), "l1.mlp.shared.sg": (1, 24)}
    for e in range(3):
        shapes.update({"l1.mlp.e%d.gate" % e: (10, 24), "l1.mlp.e%d.up" % e: (10, 24), "l1.mlp.e%d.down" % e: (24, 10)})
    W = {k: 0.4 * torch.randn(*v, generator=g) for k, v in shapes.items()}
    toks = np.random.RandomState(1).randint(0, 50, 19).tolist()
    whole = ref.forward(cfg, W, toks).numpy()
    assert np.array_equal(whole, ref.forward(cfg, W, toks).numpy())
    for n in (1, 2, 7, 18):
        assert np.allclose(ref.forward(cfg, W, toks[:n]).numpy(), whole[:n], rtol=0, atol=1e-12)
