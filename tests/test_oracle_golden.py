"""The plain-C oracle against the frozen PyTorch-CPU fixtures (CPU only)."""
import numpy as np
import pytest

from oracle import oracle
from tests.helpers import assert_close


def _ce_names(golden):
    return sorted({k.split("/")[0] for k in golden.files if k.startswith("ce_")})


def test_ce_cases_present(golden):
    assert len(_ce_names(golden)) >= 20


@pytest.mark.parametrize("idx", range(32))
def test_cross_entropy_matches_golden(golden, idx):
    names = _ce_names(golden)
    if idx >= len(names):
        pytest.skip("no such case")
    name = names[idx]
    red = name.split("_")[2]
    ignore_index, eps = golden[name + "/meta"]
    go = golden[name + "/grad_out"]
    loss, grad, bad = oracle.c_cross_entropy(
        golden[name + "/logits"], golden[name + "/target"], int(ignore_index), float(eps), red,
        grad_out=1.0 if red == "none" else float(go), row_grad_out=go if red == "none" else None)
    assert bad == 0
    expect = np.atleast_1d(golden[name + "/loss"])
    assert_close(loss, expect, 2e-6, 2e-6, name + " loss")
    assert_close(grad, golden[name + "/grad"], 1e-5, 2e-7, name + " grad")


def test_all_ignored_mean_is_nan(golden):
    loss, grad, _ = oracle.c_cross_entropy(golden["ce_4x10_mean_allignored/logits"], golden["ce_4x10_mean_allignored/target"])
    assert np.isnan(loss[0]) and np.isnan(golden["ce_4x10_mean_allignored/loss"])
    assert np.all(grad == 0)


def test_out_of_range_target_is_counted_not_fatal():
    x = np.zeros((3, 4), dtype=np.float32)
    loss, grad, bad = oracle.c_cross_entropy(x, np.array([1, 9, -3]), reduction="sum")
    assert bad == 2
    assert_close(loss, [np.log(4.0)], 1e-12, 0, "loss")
    assert np.all(grad[1:] == 0)


@pytest.mark.parametrize("name", ["lsm_last", "lsm_mid", "lsm_long"])
def test_log_softmax(golden, name):
    dim = int(golden[name + "/dim"][0])
    y = oracle.c_log_softmax(golden[name + "/x"], dim)
    assert_close(y, golden[name + "/y"], 2e-6, 2e-6, name)
    gi = oracle.c_log_softmax_backward(golden[name + "/grad_out"], golden[name + "/y"], dim)
    assert_close(gi, golden[name + "/grad_in"], 1e-5, 2e-6, name + " backward")


@pytest.mark.parametrize("name", ["sm_last", "sm_mid"])
def test_softmax(golden, name):
    dim = int(golden[name + "/dim"][0])
    y = oracle.c_softmax(golden[name + "/x"], dim)
    assert_close(y, golden[name + "/y"], 2e-6, 1e-8, name)
    gi = oracle.c_softmax_backward(golden[name + "/grad_out"], golden[name + "/y"], dim)
    assert_close(gi, golden[name + "/grad_in"], 2e-5, 1e-7, name + " backward")


@pytest.mark.parametrize("name", ["nll_mean", "nll_sum_w", "nll_none_w", "nll_mean_w"])
def test_nll_loss(golden, name):
    red = name.split("_")[1]
    w = golden[name + "/weight"] if name.endswith("_w") else None
    out, tw = oracle.c_nll_loss(golden[name + "/logp"], golden[name + "/target"], w, -100, red)
    assert_close(out, np.atleast_1d(golden[name + "/out"]), 2e-6, 2e-6, name)
    gi = oracle.c_nll_loss_backward(golden[name + "/grad_out"], golden[name + "/target"], 23, w, -100, red, tw)
    assert_close(gi, golden[name + "/grad_in"], 2e-6, 1e-7, name + " backward")


@pytest.mark.parametrize("name", ["nll2d_mean", "nll2d_sum_w", "nll2d_none_w", "nll2d_mean_w"])
def test_nll_loss2d(golden, name):
    red = name.split("_")[1]
    w = golden[name + "/weight"] if name.endswith("_w") else None
    logp = golden[name + "/logp"]
    out, tw = oracle.c_nll_loss_nd(logp, golden[name + "/target"], w, -100, red)
    assert_close(out, np.atleast_1d(golden[name + "/out"]), 2e-6, 2e-6, name)
    gi = oracle.c_nll_loss_nd_backward(golden[name + "/grad_out"], golden[name + "/target"], logp.shape, w, -100, red, tw)
    assert_close(gi, golden[name + "/grad_in"], 2e-6, 1e-7, name + " backward")


@pytest.mark.parametrize("name", ["bce_plain", "bce_w", "bce_pw", "bce_pw_w"])
def test_bce_with_logits(golden, name):
    pw = golden[name + "/pos_weight"] if (name + "/pos_weight") in golden.files else None
    w = golden[name + "/weight"] if (name + "/weight") in golden.files else None
    loss, grad = oracle.c_bce_with_logits(golden[name + "/x"], golden[name + "/target"], pw, w)
    assert_close(loss, golden[name + "/loss"], 2e-6, 2e-6, name)
    assert_close(np.atleast_1d(loss.mean()), np.atleast_1d(golden[name + "/mean"]), 2e-6, 2e-6, name + " mean")
    assert_close(grad * golden[name + "/grad_out"], golden[name + "/grad_in"], 4e-6, 2e-6, name + " backward")


def test_row_reductions(golden):
    x = golden["red/x"]
    assert_close(oracle.c_reduce_rows(x, "sum"), golden["red/sum"], 1e-5, 1e-5, "sum")
    assert_close(oracle.c_reduce_rows(x, "mean"), golden["red/mean"], 1e-5, 1e-6, "mean")
    assert np.array_equal(oracle.c_reduce_rows(x, "amax"), golden["red/amax"].astype(np.float64))
    assert np.array_equal(oracle.c_reduce_rows(x, "amin"), golden["red/amin"].astype(np.float64))
    xn = x.copy()
    xn[2, 5] = np.nan
    assert np.isnan(oracle.c_reduce_rows(xn, "amax")[2])


def test_activations(golden):
    x = golden["act/x"].astype(np.float64)
    go = golden["act/grad_out"].astype(np.float64)
    for key, fwd, bwd in (("gelu_erf", 6, 10), ("gelu_tanh", 7, 11), ("silu", 8, 12)):
        assert_close(oracle.c_elementwise(fwd, x), golden[f"act/{key}"], 2e-6, 2e-6, key)
        assert_close(oracle.c_elementwise(bwd, go, x), golden[f"act/{key}_bwd"], 4e-6, 2e-6, key + " backward")
    a, b = x[:, :7], x[:, 7:]
    assert_close(oracle.c_elementwise(9, a, b), golden["act/glu"], 2e-6, 2e-6, "glu")
    g = golden["act/glu_grad_out"].astype(np.float64)
    ga = oracle.c_elementwise(13, g, b)
    gb = oracle.c_elementwise(14, g, b, a)
    assert_close(np.concatenate([ga, gb], axis=1), golden["act/glu_bwd"], 4e-6, 2e-6, "glu backward")


def test_binary(golden):
    f = golden["bin/f32"].astype(np.float64)
    assert_close(oracle.c_elementwise(2, f, f.T.copy(), alpha=2.5), golden["bin/add_alpha"], 2e-6, 2e-6, "add alpha")
    assert_close(oracle.c_elementwise(3, f.T.copy(), f), golden["bin/mul_t"], 2e-6, 2e-6, "mul")


# ---- rows added later: weights with smoothing, probability targets, indexed extrema, moments, prod / nansum, div modes ----
@pytest.mark.parametrize("name", ["cew_mean", "cew_sum", "cew_none"])
def test_cross_entropy_weights_and_smoothing(golden, name):
    red = name.split("_")[1]
    go = golden[name + "/grad_out"]
    loss, grad, bad = oracle.c_cross_entropy_weighted(
        golden[name + "/logits"], golden[name + "/target"], golden[name + "/weight"], -100, 0.2, red,
        grad_out=1.0 if red == "none" else float(go), row_grad_out=go if red == "none" else None)
    assert bad == 0
    assert_close(loss, np.atleast_1d(golden[name + "/loss"]), 2e-6, 2e-6, name + " loss")
    assert_close(grad, golden[name + "/grad"], 1e-5, 2e-7, name + " grad")


def test_weighted_oracle_without_weights_is_the_plain_one(golden):
    name = "ce_6x130_mean_ign2_eps1"
    a = oracle.c_cross_entropy(golden[name + "/logits"], golden[name + "/target"], -100, 0.1, "mean")
    b = oracle.c_cross_entropy_weighted(golden[name + "/logits"], golden[name + "/target"], None, -100, 0.1, "mean")
    assert_close(b[0], a[0], 1e-14, 0, "loss")
    assert_close(b[1], a[1], 1e-12, 1e-18, "grad")


@pytest.mark.parametrize("name", ["cep_mean", "cep_sum_w", "cep_none_eps", "cep_mean_w_eps"])
def test_cross_entropy_probability_targets(golden, name):
    red = name.split("_")[1]
    go = golden[name + "/grad_out"]
    w = golden[name + "/weight"] if name + "/weight" in golden.files else None
    loss, grad = oracle.c_cross_entropy_prob(golden[name + "/logits"], golden[name + "/target"], w, float(golden[name + "/eps"][0]), red,
                                             grad_out=1.0 if red == "none" else float(go), row_grad_out=go if red == "none" else None)
    assert_close(loss, np.atleast_1d(golden[name + "/loss"]), 2e-6, 2e-6, name + " loss")
    assert_close(grad, golden[name + "/grad"], 1e-5, 2e-7, name + " grad")


@pytest.mark.parametrize("dim", [0, 1, 2])
@pytest.mark.parametrize("is_max", [True, False])
def test_indexed_extrema(golden, dim, is_max):
    values, indices = oracle.c_arg_reduce(golden["arg/x"], dim, is_max)
    key = f"arg/{'max' if is_max else 'min'}{dim}"
    assert np.array_equal(indices, golden[key + "_indices"])
    assert np.array_equal(values, golden[key + "_values"].astype(np.float64), equal_nan=True)


def test_indexed_extrema_flat_and_int(golden):
    x = golden["arg/x"][0]
    assert oracle.c_arg_reduce(x.reshape(-1), 0, True)[1] == golden["arg/argmax_flat"]
    assert oracle.c_arg_reduce(x.reshape(-1), 0, False)[1] == golden["arg/argmin_flat"]
    assert np.array_equal(oracle.c_arg_reduce(golden["arg/i32"], 1, True)[1], golden["arg/i32_argmax1"])
    v, i = oracle.c_arg_reduce(golden["arg/i32"], 1, False)
    assert np.array_equal(i, golden["arg/i32_min1_indices"]) and np.array_equal(v, golden["arg/i32_min1_values"])


@pytest.mark.parametrize("dim", [0, 1, 2])
def test_moments(golden, dim):
    x = golden["mom/x"]
    assert_close(oracle.c_moments(x, dim, 1.0, False)[0], golden[f"mom/var{dim}"], 2e-6, 1e-6, "var")
    assert_close(oracle.c_moments(x, dim, 0.0, True)[0], golden[f"mom/std{dim}_c0"], 2e-6, 1e-6, "std")
    if dim == 1:
        assert_close(oracle.c_moments(x, 1)[1], golden["mom/mean1"], 2e-6, 1e-6, "mean")
    assert_close(oracle.c_moments(x.reshape(-1), 0)[0], golden["mom/var_all"], 2e-6, 1e-6, "var of all")


def test_div_rounding_modes(golden):
    a, b = golden["div/a"], golden["div/b"]
    for code, key in ((38, "trunc"), (39, "floor")):
        got = oracle.c_elementwise(code, a, b)
        want = golden["div/" + key].astype(np.float64)
        assert np.array_equal(got, want, equal_nan=True), key
        assert np.array_equal(np.signbit(got), np.signbit(want)), key + ": sign of zero"
    assert np.array_equal(oracle.c_div_int(golden["div/ia"], golden["div/ib"], False), golden["div/itrunc"])
    assert np.array_equal(oracle.c_div_int(golden["div/ia"], golden["div/ib"], True), golden["div/ifloor"])


# ---- the Philox stream behind the device generator ------------------------------------------------------------------------
# Known answers published with the algorithm (Random123's kat_vectors, philox4x32 with 10 rounds): counter, key, output.
PHILOX_KAT = [
    ((0x00000000,) * 4, (0x00000000,) * 2, (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)),
    ((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2, (0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)),
    ((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0), (0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1)),
]


@pytest.mark.parametrize("counter,key,want", PHILOX_KAT)
def test_philox_known_answers(counter, key, want):
    got = oracle.philox4x32_10(np.array([counter], np.uint32), key)[0]
    assert tuple(int(v) for v in got) == want


def test_stream_layout_and_offsets():
    seed = (0x299F31D0 << 32) | 0xA4093822
    # group g of the stream at offset 4 * b is the block with counter {lo(b), hi(b), lo(g), hi(g)}
    block = (0x85A308D3 << 32) | 0x243F6A88
    ctr = np.array([[0x243F6A88, 0x85A308D3, 5, 0]], np.uint32)
    assert np.array_equal(oracle.rng_words(24, seed, 4 * block)[5], oracle.philox4x32_10(ctr, (0xA4093822, 0x299F31D0))[0])
    # consecutive fills (offset += 4) do not share a block; 8-byte element types take two words per element
    a, b = oracle.rng_words(64, 7, 0), oracle.rng_words(64, 7, 4)
    assert not np.intersect1d(a.reshape(-1), b.reshape(-1)).size
    assert oracle.rng_words(10, 7, 0, per_group=2).shape == (5, 4)


def test_distributions_of_the_stream():
    n = 1 << 18
    u = oracle.rng_uniform(n, 11, 0)
    assert u.dtype == np.float32 and u.min() >= 0 and u.max() < 1 and abs(u.mean() - 0.5) < 4e-3
    z = oracle.rng_normal(n, 11, 4)
    assert np.isfinite(z).all() and abs(z.mean()) < 1e-2 and abs(z.std() - 1) < 1e-2
    r = oracle.rng_integer(n, 11, 8, -3, 10)
    assert r.min() == -3 and r.max() == 6 and np.all(np.bincount(r + 3) > n / 10 * 0.9)
    assert abs(oracle.rng_bernoulli(n, 11, 12, 0.3).mean() - 0.3) < 5e-3
    assert np.array_equal(oracle.rng_dropout_keep(n, 11, 12, 0.3), ~oracle.rng_bernoulli(n, 11, 12, 0.3))
    w = oracle.rng_integer(1000, 11, 16, -(1 << 63), 0, wide=True)
    assert w.dtype == np.int64 and (w < 0).any() and (w > 0).any()
