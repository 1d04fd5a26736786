"""Operators of ops/extra_ops.py against NumPy restatements."""
import numpy as np
import pytest
import torch

import mxnet_b200 as mx
from mxnet_b200 import nd
from mxnet_b200.ops import registry


def _run(name, *tensors, **attrs):
    out = registry.get(name).fn(*[torch.as_tensor(t) if t is not None else None for t in tensors], **attrs)
    return [o.cpu().numpy() for o in out] if isinstance(out, (tuple, list)) else out.cpu().numpy()


def test_scalar_variants_of_binary_functions():
    x = np.array([-2.5, 0.5, 3.0], dtype='float32')
    np.testing.assert_allclose(_run('_npi_arctan2_scalar', x, scalar=2.0), np.arctan2(x, 2.0), rtol=1e-6)
    np.testing.assert_allclose(_run('_npi_rarctan2_scalar', x, scalar=2.0), np.arctan2(2.0, x), rtol=1e-6)
    np.testing.assert_allclose(_run('_npi_copysign_scalar', x, scalar=-1.0), np.copysign(x, -1.0))
    np.testing.assert_allclose(_run('_npi_rcopysign_scalar', x, scalar=4.0), np.copysign(4.0, x))
    np.testing.assert_allclose(_run('_npi_fmax_scalar', x, scalar=1.0), np.fmax(x, 1.0))
    np.testing.assert_allclose(_run('_npi_fmin_scalar', x, scalar=1.0), np.fmin(x, 1.0))
    np.testing.assert_allclose(_run('_npi_fmod_scalar', x, scalar=2.0), np.fmod(x, 2.0))
    np.testing.assert_allclose(_run('_npi_rfmod_scalar', x, scalar=2.0), np.fmod(2.0, x))
    np.testing.assert_allclose(_run('_npi_ldexp_scalar', x, scalar=3.0), np.ldexp(x, 3))
    np.testing.assert_allclose(_run('_npi_rldexp_scalar', np.array([1., 2.], 'float32'), scalar=3.0), 3.0 * 2.0 ** np.array([1., 2.]))
    np.testing.assert_allclose(_run('_npi_logaddexp_scalar', x, scalar=1.0), np.logaddexp(x, 1.0), rtol=1e-6)
    i = np.array([12, 18, 7], dtype='int64')
    np.testing.assert_array_equal(_run('_npi_gcd_scalar', i, scalar=6), np.gcd(i, 6))
    np.testing.assert_array_equal(_run('_npi_lcm_scalar', i, scalar=6), np.lcm(i, 6))
    np.testing.assert_array_equal(_run('_npi_bitwise_left_shift_scalar', i, scalar=2), i << 2)
    np.testing.assert_array_equal(_run('_npi_rbitwise_right_shift_scalar', np.array([1, 2]), scalar=16), 16 >> np.array([1, 2]))
    np.testing.assert_allclose(_run('_npi_deg2rad', x), np.deg2rad(x), rtol=1e-6)
    np.testing.assert_allclose(_run('_npi_rad2deg', x), np.rad2deg(x), rtol=1e-6)


def test_where_mask_assign_indexing_and_splits():
    c = np.array([[1, 0], [0, 1]], dtype='float32')
    x = np.array([[1., 2.], [3., 4.]], dtype='float32')
    np.testing.assert_allclose(_run('_npi_where_lscalar', c, x, scalar=9.0), np.where(c, 9.0, x))
    np.testing.assert_allclose(_run('_npi_where_rscalar', c, x, scalar=9.0), np.where(c, x, 9.0))
    np.testing.assert_allclose(_run('_npi_where_scalar2', c, x=1.5, y=-1.0), np.where(c, 1.5, -1.0))
    np.testing.assert_allclose(_run('_npi_boolean_mask_assign_scalar', x, c, value=0.0), np.where(c, 0.0, x))
    np.testing.assert_allclose(_run('_npi_boolean_mask_assign_tensor', x, c, np.array([7., 8.], 'float32')), [[7, 2], [3, 8]])
    np.testing.assert_allclose(_run('_npi_boolean_mask_assign_scalar', x, np.array([1, 0], 'float32'), value=5.0, start_axis=1),
                               [[5, 2], [5, 4]])
    np.testing.assert_allclose(_run('_npi_advanced_indexing', x, np.array([1, 0])), x[[1, 0]])
    np.testing.assert_allclose(_run('_npi_advanced_indexing_multiple', x, np.array([0, 1]), np.array([1, 0])), x[[0, 1], [1, 0]])
    np.testing.assert_allclose(_run('_npi_diagflat', np.array([1., 2.], 'float32'), k=1), np.diagflat([1., 2.], 1))
    a = np.arange(24, dtype='float32').reshape(2, 4, 3)
    for got, ref in zip(_run('_npi_hsplit', a, sections=2), np.hsplit(a, 2)):
        np.testing.assert_allclose(got, ref)
    for got, ref in zip(_run('_npi_dsplit', a, indices=(1,)), np.dsplit(a, [1])):
        np.testing.assert_allclose(got, ref)
    np.testing.assert_array_equal(_run('_npi_diag_indices_from', np.zeros((3, 3), 'float32')), np.stack(np.diag_indices_from(np.zeros((3, 3)))))
    t = torch.arange(6.)
    assert bool(registry.get('_npi_share_memory').fn(t, t[2:])) and not bool(registry.get('_npi_share_memory').fn(t, t.clone()))


def test_random_additions_have_the_right_moments():
    mx.random.seed(3)
    s = _run('_npi_normal_n', np.array([0., 10.], 'float32'), np.array([1., 2.], 'float32'), size=(20000,))
    assert s.shape == (20000, 2)
    np.testing.assert_allclose(s.mean(0), [0, 10], atol=0.1)
    np.testing.assert_allclose(s.std(0), [1, 2], rtol=0.05)
    u = _run('_npi_uniform_n', np.array([0., 2.], 'float32'), np.array([1., 6.], 'float32'), size=(20000,))
    np.testing.assert_allclose(u.mean(0), [0.5, 4.0], atol=0.05)
    b = registry.get('_random_binomial').fn(n=10, p=0.3, shape=(20000,)).cpu().numpy()
    np.testing.assert_allclose(b.mean(), 3.0, atol=0.1)
    sb = _run('_sample_binomial', np.array([10., 20.], 'float32'), np.array([0.5, 0.1], 'float32'), shape=(5000,))
    assert sb.shape == (2, 5000)
    np.testing.assert_allclose(sb.mean(1), [5.0, 2.0], atol=0.15)
    assert nd.random_binomial(n=4, p=0.5, shape=(3,)).shape == (3,)


def test_hard_sigmoid_sparse_retain_and_aliases():
    x = np.array([-5., 0., 1., 5.], 'float32')
    np.testing.assert_allclose(_run('hard_sigmoid', x, alpha=0.2, beta=0.5), np.clip(0.2 * x + 0.5, 0, 1))
    d = np.arange(12, dtype='float32').reshape(4, 3)
    out = _run('_sparse_retain', d, np.array([0, 2]))
    np.testing.assert_allclose(out[[0, 2]], d[[0, 2]])
    assert not out[[1, 3]].any()
    np.testing.assert_allclose(_run('_npx_relu', x), np.maximum(x, 0))
    np.testing.assert_allclose(_run('_npx_sigmoid', x), 1 / (1 + np.exp(-x)), rtol=1e-6)
    np.testing.assert_allclose(_run('cast_storage', d, stype='row_sparse'), d)
    np.testing.assert_allclose(nd.hard_sigmoid(nd.array(x)).asnumpy(), np.clip(0.2 * x + 0.5, 0, 1))


def test_box_encode_decode_round_trip():
    rng = np.random.RandomState(0)
    xy = rng.uniform(0, 50, (1, 6, 2))
    anchors = np.concatenate([xy, xy + rng.uniform(5, 20, (1, 6, 2))], -1).astype('float32')
    xy = rng.uniform(0, 50, (1, 3, 2))
    refs = np.concatenate([xy, xy + rng.uniform(5, 20, (1, 3, 2))], -1).astype('float32')
    samples = np.array([[1, 1, -1, 1, 0, 1]], 'float32')
    matches = np.array([[0, 2, 1, 1, 0, 2]], 'float32')
    means, stds = np.zeros(4, 'float32'), np.array([0.1, 0.1, 0.2, 0.2], 'float32')
    targets, masks = _run('_contrib_box_encode', samples, matches, anchors, refs, means, stds)
    assert targets.shape == (1, 6, 4) and masks[0, 2].sum() == 0 and masks[0, 0].sum() == 4 and not targets[0, 4].any()
    decoded = _run('_contrib_box_decode', targets, anchors, std0=0.1, std1=0.1, std2=0.2, std3=0.2, format='corner')
    pos = samples[0] > 0.5
    np.testing.assert_allclose(decoded[0][pos], refs[0][matches[0].astype(int)][pos], rtol=1e-4, atol=1e-3)


def test_intgemm_family_matches_float_product():
    rng = np.random.RandomState(1)
    x, w = rng.randn(8, 16).astype('float32'), rng.randn(4, 16).astype('float32')
    mw = _run('_contrib_intgemm_maxabsolute', w)
    np.testing.assert_allclose(mw, [np.abs(w).max()])
    wq = _run('_contrib_intgemm_prepare_weight', w, mw)
    assert wq.dtype == np.int8 and np.abs(wq).max() == 127
    np.testing.assert_array_equal(_run('_contrib_intgemm_take_weight', wq, np.array([2, 0])), wq[[2, 0]])
    scaling = np.array([mw[0] / 127.0], 'float32')
    out = _run('_contrib_intgemm_fully_connected', x, wq, scaling, None, num_hidden=4, no_bias=True)
    np.testing.assert_allclose(out, x @ w.T, atol=0.15)
    xq = _run('_contrib_intgemm_prepare_data', x, _run('_contrib_intgemm_maxabsolute', x))
    raw = _run('_contrib_intgemm_fully_connected', xq, wq, None, None, num_hidden=4, no_bias=True, out_type='int32')
    np.testing.assert_array_equal(raw, xq.astype('int32') @ wq.astype('int32').T)


def test_multi_adabelief_matches_single_updates():
    rng = np.random.RandomState(2)
    ws = [rng.randn(5).astype('float32'), rng.randn(3, 2).astype('float32')]
    gs = [rng.randn(*w.shape).astype('float32') for w in ws]
    single = []
    for w, g in zip(ws, gs):
        t = [torch.tensor(w), torch.tensor(g), torch.zeros(w.shape), torch.zeros(w.shape)]
        registry.get('_adabelief_update').fn(*t, torch.tensor(1.0), lr=0.1, wd=0.01, eta=1.0)
        single.append(t[0].numpy())
    flat = []
    for w, g in zip(ws, gs):
        flat += [torch.tensor(w), torch.tensor(g), torch.zeros(w.shape), torch.zeros(w.shape)]
    outs = registry.get('_multi_adabelief_update').fn(*flat, torch.tensor(1.0), lrs=(0.1, 0.1), wds=(0.01, 0.01), etas=(1.0, 1.0), num_weights=2)
    for o, s in zip(outs, single):
        np.testing.assert_allclose(o.numpy(), s, rtol=1e-6)


def test_quantized_additions():
    rng = np.random.RandomState(3)
    a, b = rng.randn(4, 6).astype('float32'), rng.randn(4, 6).astype('float32')

    def q(x):
        m = np.abs(x).max()
        return np.clip(np.round(x * 127 / m), -127, 127).astype('int8'), np.array([-m], 'float32'), np.array([m], 'float32')
    qa, la, ha = q(a)
    qb, lb, hb = q(b)
    out, lo, hi = _run('_contrib_quantized_elemwise_mul', qa, qb, la, ha, lb, hb)
    np.testing.assert_allclose(out.astype('float32') * hi[0] / 127, a * b, atol=0.15)
    out, lo, hi = _run('_contrib_quantized_npi_add', qa, qb, la, ha, lb, hb)
    np.testing.assert_allclose(out.astype('float32') * hi[0] / 127, a + b, atol=0.1)
    out, lo, hi = _run('_contrib_quantized_concat', qa, qb, la, ha, lb, hb, num_args=2, dim=1)
    np.testing.assert_allclose(out.astype('float32') * hi[0] / 127, np.concatenate([a, b], 1), atol=0.06)
    qd, scale, shift = _run('_contrib_quantize_asym', a)
    np.testing.assert_allclose((qd.astype('float32') - shift[0]) / scale[0], a, atol=0.02)
    g, be, mm, mv = rng.rand(6).astype('float32') + 0.5, rng.randn(6).astype('float32'), rng.randn(6).astype('float32') * 0.1, rng.rand(6).astype('float32') + 0.5
    out, lo, hi = _run('_contrib_quantized_batch_norm', qa.reshape(4, 6, 1, 1), g, be, mm, mv, la, ha, fix_gamma=False, eps=1e-5)
    ref = (a - mm) / np.sqrt(mv + 1e-5) * g + be
    np.testing.assert_allclose(out.reshape(4, 6).astype('float32') * hi[0] / 127, ref, atol=0.1)
    t, lo2, hi2 = _run('_npx_quantized_transpose', qa, la, ha, axes=(1, 0))
    np.testing.assert_array_equal(t, qa.T)


def test_random_crop_and_decoder_operators(tmp_path):
    import io
    from PIL import Image
    img = nd.array(np.random.RandomState(0).randint(0, 255, (20, 30, 3)), dtype='uint8')
    assert nd.image.random_crop(img, width=10, height=8).shape == (8, 10, 3)
    assert nd.image.random_crop(img, width=40, height=25).shape == (25, 40, 3)          # smaller images are resized up
    assert nd.image.random_resized_crop(img, width=12, height=12).shape == (12, 12, 3)
    corner = nd.image.random_crop(img, xrange=(0.0, 0.0), yrange=(1.0, 1.0), width=10, height=8).asnumpy()
    np.testing.assert_array_equal(corner, img.asnumpy()[12:, :10])
    b = io.BytesIO()
    Image.fromarray(img.asnumpy()).save(b, format='PNG')
    buf = nd.array(np.frombuffer(b.getvalue(), dtype='uint8'), dtype='uint8')
    np.testing.assert_array_equal(nd._internal._cvimdecode(buf).asnumpy(), img.asnumpy())
    path = tmp_path / 't.png'
    path.write_bytes(b.getvalue())
    np.testing.assert_array_equal(nd._internal._cvimread(filename=str(path)).asnumpy(), img.asnumpy())
    gray = nd._internal._cvimread(filename=str(path), flag=0)
    assert gray.shape == (20, 30, 1)


def test_dgl_graph_operators():
    x = np.array([[1, 0, 0, 2], [3, 0, 4, 0], [0, 5, 0, 0], [0, 6, 7, 0]], dtype='float32')
    new, old = _run('_contrib_dgl_subgraph', x, np.array([0, 1, 2]), num_args=2, return_mapping=True)
    np.testing.assert_array_equal(new, [[1, 0, 0], [2, 0, 3], [0, 4, 0]])
    np.testing.assert_array_equal(old, [[1, 0, 0], [3, 0, 4], [0, 5, 0]])
    # a complete graph on five vertices with edge ids 1..20
    g = np.zeros((5, 5), dtype='float32')
    g[~np.eye(5, dtype=bool)] = np.arange(1, 21)
    np.random.seed(0)
    vid, sub, layer = _run('_contrib_dgl_csr_neighbor_uniform_sample', g, np.array([0, 1]), num_args=2, num_hops=1, num_neighbor=2,
                           max_num_vertices=5)
    n = int(vid[-1])
    assert vid.shape == (6,) and sub.shape == (5, 5) and layer.shape == (5,) and 2 <= n <= 5
    verts = vid[:n]
    assert list(verts) == sorted(verts) and {0, 1} <= set(verts.tolist())
    assert sorted(layer[:n].tolist())[:2] == [0, 0] and (layer[n:] == -1).all()
    rows = [list(verts).index(s) for s in (0, 1)]
    for r, s in zip(rows, (0, 1)):
        picked = np.nonzero(sub[r])[0]
        assert 1 <= len(picked) <= 2 and all(sub[r, c] == g[s, c] for c in picked)      # parent edge ids on sampled edges
    prob = np.array([0.0, 0.0, 1.0, 1.0, 0.0], dtype='float32')
    vid2, sub2, pr, layer2 = _run('_contrib_dgl_csr_neighbor_non_uniform_sample', g, prob, np.array([0]), num_args=3, num_hops=1,
                                  num_neighbor=2, max_num_vertices=4)
    assert set(vid2[:int(vid2[-1])].tolist()) == {0, 2, 3}                              # only vertices with weight are drawn
    np.testing.assert_allclose(pr[:3], [0.0, 1.0, 1.0])
    compact = _run('_contrib_dgl_graph_compact', sub2, vid2, num_args=2, graph_sizes=(3,), return_mapping=False)
    assert compact.shape == (3, 3) and sorted(compact[compact != 0].tolist()) == [1.0, 2.0]


def test_quantized_rnn_follows_the_float_operator():
    from mxnet_b200.ops.nn import rnn_param_size
    rng = np.random.RandomState(5)
    T, B, I, H = 4, 2, 6, 5
    x = rng.rand(T, B, I).astype('float32')
    params = (rng.randn(rnn_param_size('lstm', 1, I, H)) * 0.3).astype('float32')
    h0, c0 = np.zeros((1, B, H), 'float32'), np.zeros((1, B, H), 'float32')
    q, scale, shift = _run('_contrib_quantize_asym', x)
    ref = _run('RNN', x, params, h0, c0, state_size=H, num_layers=1, mode='lstm')
    got = _run('_contrib_quantized_rnn', q, params, h0, c0, scale, shift, state_size=H, num_layers=1, mode='lstm')
    np.testing.assert_allclose(got, ref, atol=5e-3)
