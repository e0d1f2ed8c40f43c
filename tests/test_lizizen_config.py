"""CPU tests of the Lizizen design: configuration parsing and refusals, the spec's tensor names
and shapes, the order of layer runs with a loop, the random-weights folder, cache groups whose
pages a chunked mask gives back, the layout of attention work under a chunked mask, and the
plain implementation's own mechanisms against closed forms."""
import copy
import json

import numpy as np
import pytest
import torch

import lizizen_configs as lc
import plain_lizizen as plain
from velox_b200.cache.manager import CacheGroup, CacheManager
from velox_b200.config.model_config import ConfigError, LizizenConfig
from velox_b200.config.registry import architecture_of
from velox_b200.ops import attention_plan as ap


def parse(cfg):
    arch = architecture_of(cfg)
    return arch, arch.parse_config(cfg)


@pytest.mark.parametrize("name", list(lc.ALL))
def test_configuration_round_trip_and_tensor_names(name):
    cfg = lc.ALL[name]
    arch, typed = parse(cfg)
    assert isinstance(typed, LizizenConfig)
    again = typed.to_json_dict()
    assert again["layers"] == cfg["layers"] and again["vocab"] == cfg["vocab"] and again["width"] == cfg["width"]
    assert again.get("loop") == cfg.get("loop")
    assert arch.parse_config(again) == typed
    spec = arch.build_spec(typed)
    tensors = spec.checkpoint_tensors()
    E = cfg["width"]
    assert tensors["embed"].shape == (cfg["vocab"], E) and tensors["head"].shape == (cfg["vocab"], E)
    assert tensors["final.norm"].shape == (E,)
    for index, layer in enumerate(cfg["layers"]):
        p = f"l{index}."
        m = layer["mixer"]
        assert tensors[p + "norm1"].shape == (E,) and tensors[p + "shift"].shape == (E,)
        maps = 2 if layer["type"] == "attention_2" else 1
        assert tensors[p + "mix.q"].shape == (m["heads"] * maps * m["dim"], E)
        assert tensors[p + "mix.k"].shape == (m["kv_heads"] * maps * m["dim"], E)
        assert tensors[p + "mix.v"].shape == (m["kv_heads"] * m["vdim"], E)
        assert tensors[p + "mix.o"].shape == (E, m["heads"] * m["vdim"])
        if layer["type"] == "attention_2":
            assert tensors[p + "mix.g"].shape == (m["heads"] * m["vdim"], E)
            assert tensors[p + "mix.q.norm"].shape == (m["dim"],) and tensors[p + "mix.lk2"].shape == (m["dim"],)
            assert p + "mix.r1" not in tensors
        else:
            assert tensors[p + "mix.r1"].shape == (m["heads"],) and tensors[p + "mix.r2"].shape == (m["heads"],)
            assert p + "mix.g" not in tensors and p + "mix.q.norm" not in tensors
        if layer["mlp"] is None:
            assert not any(k.startswith(p + "mlp.") for k in tensors) and p + "norm2" not in tensors
        else:
            ff = layer["mlp"]["ff"]
            assert tensors[p + "norm2"].shape == (E,)
            assert tensors[p + "mlp.gate"].shape == (ff, E) and tensors[p + "mlp.up.b"].shape == (ff,)
            assert tensors[p + "mlp.down"].shape == (E, ff) and tensors[p + "mlp.down.b"].shape == (E,)
    # one schedule entry per layer run
    assert [entry.layer for entry in spec.schedule] == plain.run_order(cfg)


def test_order_of_layer_runs():
    _, typed = parse(lc.SMALL)
    assert typed.run_order() == (0, 1, 0, 1, 2)
    _, typed = parse(lc.WIDE)
    assert typed.run_order() == (0, 1, 2, 1, 2, 1, 2, 3)
    _, typed = parse(lc.ODD)
    assert typed.run_order() == (0, 1, 2, 3, 4)
    cfg = copy.deepcopy(lc.ODD)
    cfg["loop"] = {"start": 3, "stop": 5, "times": 2}
    assert parse(cfg)[1].run_order() == (0, 1, 2, 3, 4, 3, 4)
    cfg["loop"] = None
    assert parse(cfg)[1].run_order() == (0, 1, 2, 3, 4)


def test_refusals():
    base = lc.SMALL
    def broken(edit):
        cfg = copy.deepcopy(base)
        edit(cfg)
        return cfg
    cases = [
        lambda c: c["layers"][0].update(type="attention_3"),
        lambda c: c["layers"][0]["mixer"].update(heads=3),                        # not a multiple of kv_heads
        lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18),                 # more than dim
        lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7),                  # odd
        lambda c: c["layers"][0]["mixer"].update(softcap=-1.0),
        lambda c: c["layers"][0]["mixer"].update(q_temp={"coef": 0.1, "every": 2}),  # not a key of this mixer
        lambda c: c["layers"][1]["mixer"].update(mask={"size": 5}),               # not a key of this mixer
        lambda c: c["layers"][1]["mixer"].update(softcap=3.0),
        lambda c: c["layers"][1]["mixer"]["q_temp"].update(every=0),
        lambda c: c["layers"][0]["mlp"].update(kind="moe"),
        lambda c: c["layers"][0]["mlp"].update(limit=0.0),
        lambda c: c["loop"].update(stop=4),
        lambda c: c["loop"].update(start=2, stop=1),
        lambda c: c["loop"].update(times=0),
        lambda c: c.pop("norm"),
        lambda c: c.update(layers=[]),
    ]
    for index, edit in enumerate(cases):
        with pytest.raises(ConfigError):
            parse(broken(edit))
            pytest.fail(f"case {index} was accepted")


def test_random_weights_folder(tmp_path):
    from safetensors.torch import load_file

    from velox_b200.weights import write_random_model

    folder = str(tmp_path / "m")
    spec = write_random_model(folder, lc.SMALL, seed=4, dtype="bfloat16")
    tensors = load_file(folder + "/model.safetensors")
    assert set(tensors) == set(spec.checkpoint_tensors())
    assert float(tensors["l0.shift"].min()) >= 0 and float(tensors["l0.shift"].max()) <= 0.8
    assert float(tensors["l1.mix.r2"].min()) > 0
    written = json.load(open(folder + "/config.json"))
    assert written["layers"] == lc.SMALL["layers"] and written["loop"] == lc.SMALL["loop"]
    weights = {k: v.float().numpy() for k, v in tensors.items()}
    assert np.isfinite(plain.forward(lc.SMALL, weights, [3, 1, 4, 1, 5, 9, 2, 6])).all()


def test_pages_before_the_running_chunk_are_given_back():
    groups = [CacheGroup("all", None), CacheGroup("c", None, chunk=10), CacheGroup("one", None, chunk=1)]
    cache = CacheManager(groups, num_pages=40, page_size=4, max_num_seqs=2)
    seq = cache.new_sequence("a")
    assert cache.append_slots(seq, 30)
    cache.advance(seq, 30)
    # the next query is at 30, the first key of its chunk: blocks 0..6 hold keys below 28
    assert seq.tables[0].count(0) == 0
    assert [i for i, page in enumerate(seq.tables[1]) if page == 0] == [0, 1, 2, 3, 4, 5, 6]
    assert [i for i, page in enumerate(seq.tables[2]) if page == 0] == [0, 1, 2, 3, 4, 5, 6]
    cache.assert_consistent()
    assert cache.append_slots(seq, 9)
    cache.advance(seq, 9)
    # the next query is at 39 and still sees keys 30..38: block 7 (keys 28..31) stays
    assert seq.tables[1][7] != 0 and seq.tables[1][6] == 0
    assert seq.tables[2][8] == 0 and seq.tables[2][9] != 0
    cache.assert_consistent()
    cache.free(seq)
    assert cache.num_free_pages() == cache.num_total_pages
    for alloc in cache.allocators:
        alloc.assert_consistent()
        assert alloc.num_used == 0


def test_layout_of_work_under_a_chunked_mask():
    opt = ap.PlanOptions(num_kv_heads=2, group=2, window=None, use_f32=True, chunk=10)
    plan = ap.plan_attention([1, 25, 3], [50, 25, 9], opt)
    spans = {}
    for i in plan.items[ap.KIND_F32]:
        spans.setdefault(int(i[0]), []).append((int(i[1]), int(i[3]), int(i[4])))
    # the decoded token at position 49 sees keys 40..49
    assert [(lo, hi) for _, lo, hi in spans[0]] == [(40, 50)]
    # tiles of a portion start at the chunk of their first token and end behind their last
    for row_begin, lo, hi in spans[1]:
        first_token = row_begin // opt.group
        assert lo == first_token // 10 * 10 and hi > first_token
    # a portion inside the first chunk sees it from key 0
    assert all(lo == 0 for _, lo, _ in spans[2])
    kind, padded, _, _ = ap.plan_single_tokens(np.array([50, 3, 11, 10]), 4, 1, opt)
    assert [(int(i[3]), int(i[4])) for i in padded[:4]] == [(40, 50), (0, 3), (10, 11), (0, 10)]


def test_plain_mechanisms():
    rng = np.random.default_rng(0)
    # the shift: all of the row before at 1, nothing of it at 0, zeros before the first row
    h = rng.normal(size=(4, 3))
    assert np.allclose(plain.token_shift(h, np.ones(3))[1:], h[:-1]) and np.allclose(plain.token_shift(h, np.ones(3))[0], 0)
    assert np.allclose(plain.token_shift(h, np.zeros(3)), h)
    # a norm weight of zero leaves unit rows
    assert np.allclose(np.mean(plain.norm_around_zero(h, np.zeros(3), 0.0) ** 2, -1), 1.0)
    # the temperature grows by steps of `every` positions, the first of which is one short
    t = plain.query_temperature(np.arange(9.0), 0.5, 4)
    assert np.allclose(t[:3], 1.0) and np.allclose(t[3:7], 1.0 + 0.5 * np.log(2.0)) and np.allclose(t[7:], 1.0 + 0.5 * np.log(3.0))
    # the distance bias is 0 on the diagonal and r1 ln(1 + r2 d) below it
    b = plain.distance_bias(2.0, 0.5, 5)
    assert b[3, 3] == 0 and np.isclose(b[4, 1], 2.0 * np.log(2.5))
    # with scores of 0 over n keys every key gets 1 / (n + 1): the sink takes the rest
    p = plain.softmax_with_zero_sink(np.zeros((3, 3)), plain.causal(3))
    assert np.allclose(p[2], 1 / 4) and np.allclose(p[0], [1 / 2, 0, 0])
    # chunks are counted from position 0
    mask = plain.causal(7) & plain.same_chunk(7, 3)
    assert mask[5].tolist() == [False, False, False, True, True, True, False] and mask[6].tolist() == [False] * 6 + [True]
    # rotation keeps lengths, leaves the dims behind `dims` and position 0 alone, pairs i with i + dims / 2
    x = rng.normal(size=(5, 2, 8))
    y = plain.rotate_half(x, np.arange(5.0), 10.0, 4)
    assert np.allclose(np.linalg.norm(y, axis=-1), np.linalg.norm(x, axis=-1))
    assert np.allclose(y[..., 4:], x[..., 4:]) and np.allclose(y[0], x[0])
    one = np.zeros((2, 1, 8))
    one[:, 0, 1] = 1.0
    turned = plain.rotate_half(one, np.array([0.0, 3.0]), 10.0, 4)[1, 0]
    f1 = 10.0 ** (-2 * 1 / 4)
    assert np.isclose(turned[1], np.cos(3 * f1)) and np.isclose(turned[3], np.sin(3 * f1)) and turned[0] == 0
    # the cap bounds scores and leaves small ones alone
    assert abs(plain.softcap(np.array([1e4]), 5.0)[0] - 5.0) < 1e-9 and np.isclose(plain.softcap(np.array([1e-3]), 5.0)[0], 1e-3)
    # equal maps and lambda 1 would cancel: the unit norm then divides by sqrt(eps); lambda from zeros is diff
    W = {"lq1": np.zeros(4), "lk1": np.zeros(4), "lq2": np.zeros(4), "lk2": np.zeros(4)}
    assert np.isclose(plain.differential_lambda(W, "", 0.3), 0.3)
    # the feed-forward's clamps: a gate far above the limit acts as the limit, a far negative up as -limit
    Wf = {"gate": np.eye(2), "gate.b": np.array([50.0, 0.2]), "up": np.eye(2), "up.b": np.array([-50.0, 0.1]),
          "down": np.eye(2), "down.b": np.zeros(2)}
    out = plain.feed_forward(np.zeros((1, 2)), Wf, "", {"ff": 2, "limit": 1.5})[0]
    assert np.isclose(out[0], 1.5 * plain.sigmoid(1.702 * 1.5) * (-1.5 + 1.0))
    assert np.isclose(out[1], 0.2 * plain.sigmoid(1.702 * 0.2) * 1.1)
