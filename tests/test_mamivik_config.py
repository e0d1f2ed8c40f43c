"""The Mamivik design without a GPU: its configuration, its spec, its checkpoint names and shapes,
what its layers ask of the cache manager, and the plain implementation's own mechanisms against
closed forms."""
import copy
import math

import numpy as np
import pytest
import torch

import mamivik_configs as mc
import plain_mamivik as plain


def _arch(cfg):
    from velox_b200.config.registry import architecture_of

    return architecture_of(cfg)


@pytest.mark.parametrize("name", list(mc.ALL))
def test_configuration_is_read_and_written_back(name):
    cfg = mc.ALL[name]
    arch = _arch(cfg)
    typed = arch.parse_config(cfg)
    again = typed.to_json_dict()
    assert again["layers"] == cfg["layers"]
    assert again["canon"] == cfg["canon"] and again["norm"] == cfg["norm"]
    assert (again["vocab"], again["width"]) == (cfg["vocab"], cfg["width"])
    assert arch.parse_config(again) == typed


def test_what_the_configuration_refuses():
    from velox_b200.config.model_config import ConfigError

    arch = _arch(mc.SMALL)

    def broken(change):
        cfg = copy.deepcopy(mc.SMALL)
        change(cfg)
        with pytest.raises(ConfigError):
            arch.parse_config(cfg)

    broken(lambda c: c["layers"][0].update(type="attention"))
    broken(lambda c: c["layers"][0]["mixer"]["left"].update(vdim=24))          # the values are the keys
    broken(lambda c: c["layers"][0]["mixer"]["left"].update(heads=3))          # 3 heads on 2 KV heads
    broken(lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7))
    broken(lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=32))
    broken(lambda c: c["layers"][0]["mixer"].pop("left_scale"))
    broken(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=10))           # more than the rotated part has
    broken(lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].update(factor=0.0))
    broken(lambda c: c["layers"][1]["mixer"].pop("q_rank"))
    broken(lambda c: c["layers"][1]["mixer"]["mask"].update(size=0))
    broken(lambda c: c["layers"][0]["mlp"].update(kind="experts"))
    broken(lambda c: c.pop("canon"))
    broken(lambda c: c["canon"].update(taps=0))
    broken(lambda c: c.update(layers=[]))


def test_tensor_names_and_shapes():
    spec = mc.build_spec(mc.SMALL, decay_rank=5)
    tensors = {name: tuple(src.shape) for name, src in spec.checkpoint_tensors().items()}
    assert tensors["embed"] == (120, 64) and tensors["head"] == (120, 64) and tensors["final.norm"] == ()
    assert tensors["l0.norm1"] == () and tensors["l0.norm2"] == () and tensors["l0.canon1"] == (64, 3)
    assert "l1.norm2" not in tensors and "l1.mlp.gate" not in tensors       # a layer without feed-forward
    assert tensors["l0.mix.left.q"] == (64, 64) and tensors["l0.mix.left.q.b"] == (64,)
    assert tensors["l0.mix.left.k"] == (32, 64) and tensors["l0.mix.left.k.b"] == (32,)
    assert "l0.mix.left.v" not in tensors and tensors["l0.mix.left.o"] == (64, 64)
    for name in ("r", "k", "v", "g", "a"):
        assert tensors["l0.mix.right." + name] == (32, 64)
    assert tensors["l0.mix.right.w1"] == (5, 64) and tensors["l0.mix.right.w2"] == (32, 5)
    assert tensors["l0.mix.right.w0"] == (32,) and tensors["l0.mix.right.a.b"] == (32,)
    assert tensors["l0.mix.right.norm"] == (32,) and tensors["l0.mix.right.o"] == (64, 32)
    assert tensors["l1.mix.dq"] == (24, 64) and tensors["l1.mix.dq.norm"] == (24,)
    assert tensors["l1.mix.uq"] == (3 * 24, 24) and tensors["l1.mix.dkv"] == (40, 64)
    assert tensors["l1.mix.dkv.norm"] == (32,) and tensors["l1.mix.uk"] == (48, 32) and tensors["l1.mix.uv"] == (72, 32)
    assert tensors["l1.mix.sink"] == (3,) and tensors["l1.mix.g"] == (72, 64) and tensors["l1.mix.o"] == (64, 72)
    assert tensors["l0.mlp.gate"] == (40, 64) and tensors["l0.mlp.up"] == (40, 64) and tensors["l0.mlp.down"] == (64, 40)


def test_sizes_that_only_the_checkpoint_gives(tmp_path):
    """The inner size of the decay's small matrices is read from a tensor's shape."""
    from velox_b200.config.registry import architecture_of
    from velox_b200.weights.loader import Checkpoint, check_checkpoint

    folder = str(tmp_path / "model")
    mc.write_folder(folder, mc.ODD, mc.make_weights(mc.ODD, seed=1, decay_rank=5))
    arch = architecture_of(mc.ODD)
    typed = arch.parse_config(mc.ODD)
    checkpoint = Checkpoint(folder)
    sizes = arch.checkpoint_sizes(typed, lambda name: checkpoint.shape(name) if name in checkpoint else None)
    assert sizes == {"decay_ranks": {2: 5, 3: 5}}
    check_checkpoint(checkpoint, arch.build_spec(typed, **sizes))
    from velox_b200.weights.loader import WeightError

    with pytest.raises(WeightError):
        check_checkpoint(checkpoint, arch.build_spec(typed))


def test_random_weights_folder(tmp_path):
    from helpers import read_config, read_tensors, write_model

    folder = str(tmp_path / "random")
    write_model(folder, mc.SMALL, seed=3, dtype="bfloat16")
    tensors = read_tensors(folder)
    spec = mc.build_spec(mc.SMALL)
    assert set(tensors) == set(spec.checkpoint_tensors())
    assert tensors["l0.norm1"].shape == () and tensors["l0.canon1"].shape == (64, 3)
    assert read_config(folder)["layers"] == mc.SMALL["layers"]
    logits = plain.forward(mc.SMALL, mc.as_numpy(tensors), [1, 2, 3, 4, 5])
    assert np.isfinite(logits).all()


def test_parts_and_what_they_ask_of_the_cache():
    spec = mc.build_spec(mc.WIDE, decay_rank=16)
    kinds = [layer.mixer.kind for layer in spec.layers]
    assert kinds == ["latent_attention", "side_by_side", "side_by_side", "latent_attention"]
    assert all(layer.block == "pre_norm" and layer.block_params == {"input_conv": True} for layer in spec.layers)
    assert spec.layers[2].feed_forward is None and "feed_forward" not in spec.layers[2].norms
    latent = spec.layers[0].mixer.params
    assert (latent["window"], latent["query_rank"], latent["gate"], latent["sink"]) == (150, 72, "element", True)
    both = spec.layers[1].mixer.params
    assert both["join"] == "weighted_sum" and (both["left_scale"], both["right_scale"]) == (1.4, 0.8)
    assert both["left"]["params"]["values_from_keys"] and both["left"]["params"]["window"] == 200
    assert both["right"]["params"]["decay_scale"] == pytest.approx(math.exp(-0.5))
    ff = spec.layers[0].feed_forward.params
    assert ff["alpha"] == pytest.approx(2 * math.sqrt(2 / math.pi)) and ff["cubic"] == 0.044715 and not ff["biases"]
    assert spec.layers[0].position.kind == "rotary_half" and spec.layers[0].position.params["scaling"]["factor"] == 4.0
    assert spec.layers[1].position.params["scaling"] is None and spec.layers[1].position.params["rotary_dim"] == 32


def test_windows_give_pages_back():
    """A request's pages behind its windows go back to the pool: one cache group per window."""
    from velox_b200.cache.manager import CacheGroup, CacheManager

    groups = [CacheGroup(name="window_7", window=7), CacheGroup(name="window_33", window=33)]
    cache = CacheManager(groups, num_pages=40, page_size=4, max_model_len=200, max_num_seqs=2)
    seq = cache.new_sequence("a")
    assert cache.acquire_slot(seq)
    held = []
    for step in range(30):
        assert cache.append_slots(seq, 5)
        cache.advance(seq, 5)
        cache.assert_consistent()
        held.append(cache.num_total_pages - cache.num_free_pages())
    assert max(held[10:]) <= (7 + 5) // 4 + 2 + (33 + 5) // 4 + 2
    cache.free(seq)
    cache.release_slot(seq)
    assert cache.num_free_pages() == cache.num_total_pages


# ------------------------------------------------------------------ the plain mechanisms themselves
def test_plain_convolution_and_norm():
    h = np.arange(12, dtype=np.float64).reshape(4, 3) + 1.0
    w = np.array([[0.5, 2.0], [0.0, 1.0], [1.0, 0.0]])            # taps = 2: column 1 is the token itself
    out = plain.causal_conv(h, w)
    assert np.allclose(out[0], [2.0 * 1, 2.0, 0.0])
    assert np.allclose(out[2], [0.5 * 4 + 2.0 * 7, 8.0, 6.0])
    x = np.array([[3.0, 4.0]])
    assert np.allclose(plain.rms_unit(x, 0.0), x / math.sqrt(12.5))
    assert np.allclose(plain.rms_unit(x, 1.5), x / math.sqrt(14.0))


def test_plain_rotation_and_stretching():
    rot = {"base": 100.0, "dims": 4}
    x = np.array([[[1.0, 2.0, 3.0, 4.0, 5.0]]])
    out = plain.rotate_halves(x, rot, [3])
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    assert np.allclose(out[0, 0], [math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
                                   3 * math.cos(a0) + math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1), 5.0])
    assert np.allclose(plain.rotate_halves(x, rot, [0]), x)
    f, magnitude = plain.frequencies({"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}})
    plain_f = 10000.0 ** (-2.0 * np.arange(4) / 8)
    assert magnitude == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert f[0] == pytest.approx(plain_f[0]) and f[-1] == pytest.approx(plain_f[-1] / 4.0)   # fast pairs stay, slow ones stretch
    assert np.all(f <= plain_f + 1e-15) and np.all(f >= plain_f / 4.0 - 1e-15)


def test_plain_window_and_sink():
    mask = plain.window_mask(6, 3)
    assert mask[5].tolist() == [False, False, False, True, True, True] and mask[1].tolist() == [True, True, False, False, False, False]
    scores = np.zeros((1, 2, 2))
    values = np.array([[[1.0], [3.0]]])
    out = plain.attend(scores, plain.window_mask(2, 2), values, sink=np.array([0.0]))
    assert np.allclose(out[0, :, 0], [0.5, 4.0 / 3.0])                 # the sink counts once and carries no value
    out = plain.attend(scores, plain.window_mask(2, 2), values, sink=np.array([-1e9]))
    assert np.allclose(out[0, :, 0], [1.0, 2.0])


def test_plain_delta_rule_against_closed_forms():
    one = np.ones((1, 2))
    k = np.array([[3.0, 4.0]])
    v = np.array([[2.0, -1.0, 0.5]])
    # from the zero state only k v^T is left
    out, S = plain.delta_rule_states(np.array([[1.0, 0.0]]), k, v, 0.5 * one, 0.3 * one)
    assert np.allclose(S, np.outer(k[0], v[0])) and np.allclose(out[0], 3.0 * v[0])
    # a removal rate of 1 and no decay take the key's direction out of the old state before the new pair is written
    S0 = np.array([[1.0, 2.0, 3.0], [0.5, -1.0, 4.0]])
    u = k[0] / 5.0
    _, S1 = plain.delta_rule_states(one, k, 0.0 * v, one, one, S=S0)
    assert np.allclose(u @ S1, 0.0, atol=1e-6)
    # decay alone
    _, S2 = plain.delta_rule_states(one, 0.0 * k, v, np.array([[0.5, 0.25]]), 0.0 * one, S=S0)
    assert np.allclose(S2, S0 * np.array([[0.5], [0.25]]))


def test_plain_gelu_is_the_gated_sigmoid_form():
    z = np.linspace(-6, 6, 101)
    alpha, cubic = 2.0 * math.sqrt(2.0 / math.pi), 0.044715
    assert np.allclose(plain.gelu_tanh(z), z * plain.sigmoid(alpha * (z + cubic * z ** 3)), atol=1e-12)
