"""The Vobusun configuration on the CPU: keys and errors, the spec it yields (parts, tensor names, run order of layers that
run another layer's weights), random model folders read back, and properties of the plain implementation's mechanisms."""

import copy
import json
import os

import pytest
import torch

import plain_vobusun as P
import vobusun_models as M
from dryft_b200.config import ConfigError, VobusunConfig, config_from_dict, preset
from dryft_b200.weights import Checkpoint, expected_tensors, write_random_model


def test_every_key_is_read_and_round_trips():
    for name, raw in M.CONFIGS.items():
        cfg = config_from_dict(raw)
        assert isinstance(cfg, VobusunConfig)
        assert cfg.to_dict() == raw, name
        spec = cfg.model_spec()
        assert len(spec.schedule) == len(raw["layers"])
        own = [i for i, l in enumerate(raw["layers"]) if l.get("weights_of") is None]
        assert len(spec.layers) == len(own)
        for st, l in zip(spec.schedule, raw["layers"]):
            assert spec.layers[st.layer].mixer.kind == l["type"]
            assert st.cache_from is None          # a state of its own, whoever's weights it runs


def test_tensor_names_and_shapes_are_the_tests_own_weights():
    for name, raw in M.CONFIGS.items():
        want = {k: tuple(v.shape) for k, v in M.draw_weights(raw, 1).items()}
        exp = expected_tensors(config_from_dict(raw).model_spec())
        got = {k: tuple(v.shape) for k, v in exp.items() if not v.optional or k in want}
        assert got == want, name


def test_a_layer_that_runs_anothers_weights_has_no_tensors_and_may_chain():
    ls = [M.rglru(), M.retention()]
    ls += [M.again(ls, 1)]
    ls += [dict(ls[2], weights_of=2)]            # runs layer 2, which runs layer 1
    cfg = config_from_dict(M.config(ls))
    assert [cfg.weights_layer(i) for i in range(4)] == [0, 1, 1, 1]
    spec = cfg.model_spec()
    assert [s.layer for s in spec.schedule] == [0, 1, 1, 1]
    assert not any(n.startswith(("l2.", "l3.")) for n in expected_tensors(spec))


@pytest.mark.parametrize("edit, text", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0].update(type="attention"), "not a mixer"),
    (lambda c: c["layers"][1]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=2), "rot_dim"),
    (lambda c: c["layers"][0]["mixer"].update(blocks=5), "blocks"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "feed-forward"),
    (lambda c: c["layers"][4].update(weights_of=4), "weights_of"),
    (lambda c: c["layers"][4].update(weights_of=1), "differs"),
    (lambda c: c.update(streams=0), "streams"),
])
def test_errors_name_the_key(edit, text):
    raw = copy.deepcopy(M.CONFIGS["mixed"])
    edit(raw)
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert text in str(e.value)


def test_random_model_folder_reads_back(tmp_path):
    raw = M.CONFIGS["mixed"]
    d = write_random_model(raw, 3, str(tmp_path / "m"))
    assert json.load(open(os.path.join(d, "config.json"))) == raw
    spec = config_from_dict(raw).model_spec()
    ck = Checkpoint(d)
    ck.check(expected_tensors(spec))
    mix = ck.read("l1.hc1.mix").float()
    assert (mix.diagonal() > 0.5).all()           # mixing matrices are drawn around the identity
    # the plain implementation runs on what the product wrote: finite logits
    from safetensors.torch import load_file

    lg = P.forward(raw, load_file(os.path.join(d, "model.safetensors")), [1, 2, 3, 4, 5])
    assert torch.isfinite(lg).all()


def test_presets_parse():
    for name in ("vobusun-tiny", "vobusun-1k", "vobusun-2k"):
        cfg = config_from_dict(preset(name))
        assert cfg.model_spec().architecture == "Vobusun"
        assert cfg.matmul_flops_per_token() > 0 and cfg.weight_bytes_per_decode_step(2) > 0


# ----------------------------------------------------------------------------- the plain mechanisms themselves
def test_plain_pair_rows():
    assert P.bigram_rows([4, 9, 9], 7, 3, 2) == [7, (4 * 3 + 9 * 2) % 7, (9 * 3 + 9 * 2) % 7]


def test_plain_rotations_keep_lengths_and_differ_in_layout():
    x = torch.randn(5, 2, 8, dtype=torch.float64)
    pos = torch.arange(5)
    a, b = P.rotate(x, pos, 6, 100.0, False), P.rotate(x, pos, 6, 100.0, True)
    assert torch.allclose(a.norm(dim=-1), x.norm(dim=-1)) and torch.allclose(b.norm(dim=-1), x.norm(dim=-1))
    assert torch.equal(a[..., 6:], x[..., 6:]) and torch.equal(a[0], x[0])
    assert not torch.allclose(a[1:], b[1:])
    # relative: the dot product of two rotated vectors depends on the distance only
    q, k = torch.randn(1, 8, dtype=torch.float64), torch.randn(1, 8, dtype=torch.float64)
    d1 = (P.rotate(q, torch.tensor([9]), 8, 50.0, True) * P.rotate(k, torch.tensor([4]), 8, 50.0, True)).sum()
    d2 = (P.rotate(q, torch.tensor([105]), 8, 50.0, True) * P.rotate(k, torch.tensor([100]), 8, 50.0, True)).sum()
    assert torch.allclose(d1, d2)


def test_plain_retention_is_the_decayed_sum():
    raw = M.CONFIGS["ret"]
    t = {k: v for k, v in M.draw_weights(raw, 2).items()}
    m = dict(raw["layers"][0]["mixer"])
    m.pop("rot")
    T = 9
    h = torch.randn(T, raw["width"], dtype=torch.float64)
    got = P.retention(m, "l0.mix.", t, h, 1e-5)
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ t["l0.mix.q"].double().T).reshape(T, H, d)
    k = (h @ t["l0.mix.k"].double().T).reshape(T, H, d) * d ** -0.5
    v = (h @ t["l0.mix.v"].double().T).reshape(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=torch.float64)
    for i in range(T):
        for j in range(i + 1):
            for hd in range(H):
                o[i, hd] += m["decay"][hd] ** (i - j) * (q[i, hd] @ k[j, hd]) * v[j, hd]
    g = h @ t["l0.mix.g"].double().T
    want = (P.unit_rms(o, 1e-5).reshape(T, -1) * g * torch.sigmoid(g)) @ t["l0.mix.o"].double().T
    assert torch.allclose(got, want, atol=1e-9)


def test_plain_window_sees_exactly_its_last_keys():
    raw = M.CONFIGS["lat"]
    t = M.draw_weights(raw, 4)
    m = raw["layers"][0]["mixer"]
    w = m["mask"]["size"]
    h = torch.randn(w + 6, raw["width"], dtype=torch.float64)
    full = P.latent_attention(m, "l0.mix.", t, h, 1e-5)
    h2 = h.clone()
    h2[0] += 5.0                                   # a key that position w - 1 still sees and position w does not
    moved = P.latent_attention(m, "l0.mix.", t, h2, 1e-5)
    assert not torch.allclose(full[w - 1], moved[w - 1])
    assert torch.allclose(full[w:], moved[w:])
