"""CPU tests of the Tevovik design's host side: its configuration (keys, errors that name the key, the spec it
yields, the tensors the spec expects), the registry's choice by ``architecture``, random model folders, the cache's
handling of value rows of another size and of chunked visibility, and the plain implementation's own properties."""

import copy
import json

import pytest
import torch

import plain_tevovik as P
import tevovik_models as M
from dryft_b200.cache.slots import PageLedger
from dryft_b200.cache.store import KVNeed, SequenceCache
from dryft_b200.config import ConfigError, TevovikConfig, config_from_dict, known_architectures, preset
from dryft_b200.weights import Checkpoint, expected_tensors, write_random_model


def test_registry_picks_the_design_by_its_architecture_string():
    assert "Tevovik" in known_architectures()
    cfg = config_from_dict(M.CONFIGS["a"])
    assert isinstance(cfg, TevovikConfig) and cfg.num_layers == 3
    assert isinstance(config_from_dict(preset("tevovik-tiny")), TevovikConfig)


@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e", "f"])
def test_config_round_trip_and_spec(name):
    raw = M.CONFIGS[name]
    cfg = TevovikConfig.from_dict(raw)
    assert TevovikConfig.from_dict(cfg.to_dict()) == cfg
    spec = cfg.model_spec()
    assert spec.vocab_size == raw["vocab"] and spec.hidden_size == raw["width"] and len(spec.layers) == len(raw["layers"])
    for i, (ly, st) in enumerate(zip(raw["layers"], spec.schedule)):
        assert st.layer == i and st.cache_from == ly["mixer"].get("kv_from")
        assert (spec.layers[i].ffn is None) == (ly["mlp"] is None)
    # the tensors the spec expects are exactly the ones the tests' own generator writes
    assert set(expected_tensors(spec)) == set(M.draw_weights(raw, 0))
    shapes = {k: tuple(v.shape) for k, v in M.draw_weights(raw, 0).items()}
    assert {k: tuple(v.shape) for k, v in expected_tensors(spec).items()} == shapes


def test_a_layer_that_borrows_keys_has_no_key_or_value_tensors():
    names = set(expected_tensors(TevovikConfig.from_dict(M.CONFIGS["a"]).model_spec()))
    assert "l0.mix.k" in names and "l0.mix.v" in names and "l0.mix.k.norm" in names
    assert not any(n in names for n in ("l1.mix.k", "l1.mix.v", "l1.mix.k.norm"))
    assert "l1.mix.q" in names and "l1.mix.q.norm" in names and "l1.mix.g" in names
    assert "l2.norm2" not in names and not any(n.startswith("l2.mlp.") for n in names)   # no feed-forward there


def _broken(path, value):
    raw = copy.deepcopy(M.CONFIGS["a"])
    node = raw
    for key in path[:-1]:
        node = node[key]
    if value is None:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return raw


@pytest.mark.parametrize("path,value,word", [
    (("vocab",), None, "vocab"), (("width",), 0, "width"), (("norm", "eps"), -1.0, "eps"), (("embedding",), None, "embedding"),
    (("layers", 0, "type"), "recurrent", "type"), (("layers", 0, "mixer", "heads"), 3, "heads"),
    (("layers", 0, "mixer", "dim"), None, "dim"), (("layers", 1, "mixer", "kv_from"), 1, "kv_from"),
    (("layers", 1, "mixer", "kv_from"), 5, "kv_from"), (("layers", 1, "mixer", "vdim"), 8, "kv_from"),
    (("layers", 0, "mlp", "kind"), "dense", "kind"), (("layers", 0, "mlp", "router", "groups", "count"), 3, "groups"),
    (("layers", 0, "mlp", "router", "groups", "keep"), 9, "keep"), (("layers", 0, "mlp", "router", "top"), 5, "top"),
    (("layers", 0, "mixer", "mask", "size"), 0, "size"),
])
def test_config_errors_name_the_key(path, value, word):
    with pytest.raises(ConfigError) as e:
        TevovikConfig.from_dict(_broken(path, value))
    assert word in str(e.value)


def test_a_layer_cannot_borrow_from_a_borrower():
    raw = copy.deepcopy(M.CONFIGS["a"])
    raw["layers"][2] = copy.deepcopy(raw["layers"][1])
    raw["layers"][2]["mixer"]["kv_from"] = 1
    with pytest.raises(ConfigError):
        TevovikConfig.from_dict(raw)


def test_random_model_folder_loads_back(tmp_path):
    d = write_random_model(preset("tevovik-tiny"), 3, str(tmp_path / "m"), std=0.05)
    raw = json.load(open(d + "/config.json"))
    assert raw["architecture"] == "Tevovik"
    cfg = config_from_dict(raw)
    ck = Checkpoint(d)
    ck.check(expected_tensors(cfg.model_spec()))
    # norms stored around zero, lambda vectors around zero, q/k norm weights around one
    assert abs(float(ck.read("l0.norm1").float().mean())) < 0.05
    assert abs(float(ck.read("l0.mix.lq1").float().mean())) < 0.05
    assert abs(float(ck.read("l0.mix.q.norm").float().mean()) - 1.0) < 0.05
    # the plain implementation evaluates it
    from safetensors.torch import load_file

    logits = P.forward(raw, load_file(d + "/model.safetensors"), [1, 2, 3, 4, 5])
    assert logits.shape == (5, raw["vocab"]) and torch.isfinite(logits).all()


# ------------------------------------------------------------------------------------------ cache
def test_chunked_ledger_gives_back_pages_of_finished_chunks():
    led = PageLedger(n_pages=32, page_size=64, max_pages_per_slot=32, window=None, chunk=96)
    led.open(0)
    led.grow(0, 0, 500)
    assert len(led.held(0)) == 8
    # next position 500 lies in the chunk that starts at 480: pages wholly before key 480 (logical 0..6) go back
    assert led.first_live_page(500) == 7
    led.trim(0, 500)
    assert sorted(led.held(0)) == [7]
    # just inside / just outside a chunk edge
    assert led.first_live_page(479) == 384 // 64 and led.first_live_page(480) == 480 // 64
    both = PageLedger(32, 64, 32, window=100, chunk=1000)
    assert both.first_live_page(990) == (990 - 100 + 1) // 64 and both.first_live_page(1005) == 1000 // 64
    led.close(0)
    led.check()


def test_cache_entries_with_their_own_value_size_and_borrowers_with_another_view():
    cpu = torch.device("cpu")
    own = KVNeed(2, 32, None, 24, 20)
    other_view = KVNeed(2, 32, None, 24, 7)
    cache = SequenceCache([(own, None), (own, None), (other_view, None)], [None, 0, None], max_tokens=512, max_slots=2,
                          max_seq_len=512, page_size=64, dtype=torch.float32, device=cpu)
    assert cache.n_groups() == 2
    e = cache.entry(0)
    assert e.k.shape[-1] == 32 and e.v.shape[-1] == 24 and cache.entry(1).k.data_ptr() == e.k.data_ptr()
    (s,) = cache.open_sequences(1)
    cache.reserve(s, 300)
    cache.advanced(s, 300)
    assert [len(g.ledger.held(s)) for g in cache._groups] == [1, 1]       # both trim: chunk 20 -> page 4; chunk 7 -> page 4
    cache.close_sequences([s])
    # a borrower that sees keys another way than the owner keeps every page
    mixed = SequenceCache([(own, None), (other_view, None)], [None, 0], max_tokens=512, max_slots=2, max_seq_len=512,
                          page_size=64, dtype=torch.float32, device=cpu)
    (s,) = mixed.open_sequences(1)
    mixed.reserve(s, 300)
    mixed.advanced(s, 300)
    assert len(mixed._groups[0].ledger.held(s)) == 5
    mixed.close_sequences([s])
    mixed.check()


# ------------------------------------------------------------------------------------------ the plain implementation
def test_plain_router_keeps_to_the_best_groups_and_does_not_renormalise():
    g = torch.Generator().manual_seed(4)
    h = torch.randn(200, 16, generator=g, dtype=torch.float64)
    w = torch.randn(12, 16, generator=g, dtype=torch.float64)
    idx, wts = P.route(h, w, {"experts": 12, "top": 3, "groups": {"count": 4, "keep": 2}})
    s = torch.softmax(h @ w.T, -1)
    gs = s.reshape(200, 4, 3).max(-1).values
    best = gs.topk(2, dim=-1).indices
    for t in range(200):
        assert {int(i) // 3 for i in idx[t]} <= {int(b) for b in best[t]}
    assert torch.equal(wts, s.gather(1, idx)) and float(wts.sum(-1).max()) < 1.0


def test_plain_chunk_mask_makes_the_prefix_of_a_chunk_irrelevant():
    cfg = M.CONFIGS["c"]
    cfg1 = M.config([M.layer(heads=8, kv_heads=2, dim=16, vdim=16, chunk=7, diff=0.55)], width=64, vocab=130)
    t = M.draw_weights(cfg1, 2)
    a = M.prompts(cfg, [21], seed=1)[0]
    b = M.prompts(cfg, [14], seed=2)[0] + a[14:]
    la, lb = P.forward(cfg1, t, a), P.forward(cfg1, t, b)
    # positions 14..20 form a chunk of their own: with one layer nothing before position 14 can reach them
    assert torch.allclose(la[14:], lb[14:], atol=1e-12) and not torch.allclose(la[:14], lb[:14], atol=1e-3)
