"""DeviceBackend('cuda') operators against values produced by the reference's NumpyBackend."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def be():
    import versenext_b200 as vn
    vn.clear_backend_cache()
    return vn.get_backend("cuda")


def test_factory_caches_and_reports_type(be):
    import versenext_b200 as vn
    assert vn.get_backend("cuda") is be
    assert vn.get_backend("CUDA") is be
    assert be.device_type == "cuda"
    assert isinstance(be, vn.DeviceBackend)
    assert vn.get_backend("cuda:0") is not be
    vn.clear_backend_cache()
    assert vn.get_backend("cuda") is not be


def test_ops_match_reference_values(be, golden):
    g = golden("backend_reference.npz")
    tol = dict(rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(np.asarray(be.matmul(g["a"], g["b"])), g["matmul"], **tol)
    np.testing.assert_allclose(np.asarray(be.linear(g["a"], g["w"], g["bias"])), g["linear"], **tol)
    np.testing.assert_allclose(np.asarray(be.linear(g["a"], g["w"])), g["linear_nobias"], **tol)
    np.testing.assert_allclose(np.asarray(be.softmax(g["a"], dim=-1)), g["softmax"], **tol)
    np.testing.assert_allclose(np.asarray(be.softmax(g["a"], dim=1)), g["softmax_d1"], **tol)
    np.testing.assert_allclose(np.asarray(be.layernorm(g["a"], g["g"], g["beta"], eps=1e-5)), g["layernorm"], **tol)
    np.testing.assert_allclose(np.asarray(be.rmsnorm(g["a"], g["g"], eps=1e-6)), g["rmsnorm"], **tol)
    np.testing.assert_allclose(np.asarray(be.rope(g["q"], g["cos"], g["sin"])), g["rope_full"], **tol)
    np.testing.assert_allclose(np.asarray(be.rope(g["q"], g["cos"][:, :4], g["sin"][:, :4])), g["rope_half"], **tol)
    np.testing.assert_allclose(np.asarray(be.attention(g["q"], g["k"], g["v"])), g["attention"], **tol)
    np.testing.assert_allclose(np.asarray(be.attention(g["q"], g["k"], g["v"], g["mask"])), g["attention_mask"], **tol)
    qq = g["q"]
    assert be.rope(qq) is qq


def test_ops_accept_device_arrays_and_odd_shapes(be):
    rng = np.random.default_rng(0)
    a = rng.normal(0, 1, (67, 129)).astype(np.float32)
    b = rng.normal(0, 1, (129, 33)).astype(np.float32)
    ad = be.to_device(a)
    out = be.matmul(ad, b)
    assert out.shape == (67, 33)
    np.testing.assert_allclose(out.numpy(), a @ b, rtol=1e-4, atol=1e-4)
    w = rng.normal(0, 1, (5, 129)).astype(np.float32)
    np.testing.assert_allclose(be.linear(ad, w).numpy(), a @ w.T, rtol=1e-4, atol=1e-4)
    x = rng.normal(0, 3, (3, 100003)).astype(np.float32)
    sm = be.softmax(x).numpy()
    e = np.exp(x - x.max(-1, keepdims=True))
    np.testing.assert_allclose(sm, e / e.sum(-1, keepdims=True), rtol=1e-4, atol=1e-9)
    b3 = rng.normal(0, 1, (4, 6, 8)).astype(np.float32)
    c3 = rng.normal(0, 1, (8, 3)).astype(np.float32)
    np.testing.assert_allclose(be.matmul(b3, c3).numpy(), b3 @ c3, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("rows", [1, 2, 3, 5, 8, 9, 17, 32, 33])
def test_linear_with_few_rows_and_many_features(be, rows):
    """Few rows against a wide weight matrix take the weight-streaming kernel (up to 32 rows; 33 the tiled one):
    feature counts that are no multiple of the warps' groups of four, with and without bias, K = 128 and 1024."""
    rng = np.random.default_rng(rows)
    for K, N in ((128, 1027), (1024, 4098)):
        x = rng.normal(0, 1, (rows, K)).astype(np.float32)
        w = rng.normal(0, 1, (N, K)).astype(np.float32)
        b = rng.normal(0, 1, (N,)).astype(np.float32)
        want = x.astype(np.float64) @ w.T.astype(np.float64)
        np.testing.assert_allclose(be.linear(x, w).numpy(), want, rtol=2e-5, atol=2e-4)
        np.testing.assert_allclose(be.linear(x, w, b).numpy(), want + b, rtol=2e-5, atol=2e-4)


def test_shape_errors(be):
    with pytest.raises(ValueError):
        be.matmul(np.zeros((2, 3), np.float32), np.zeros((4, 5), np.float32))
    with pytest.raises(ValueError):
        be.linear(np.zeros((2, 3), np.float32), np.zeros((4, 5), np.float32))
    with pytest.raises(ValueError):
        be.attention(np.zeros((1, 2, 4), np.float32), np.zeros((1, 3, 4), np.float32), np.zeros((1, 2, 4), np.float32))
