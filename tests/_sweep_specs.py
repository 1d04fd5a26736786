"""Input specifications of the operator sweep (``test_operator_sweep.py``): for every operator that needs particular
shapes or attributes, a function ``spec(gen) -> (tensors, attrs)``; plus the names that are left out, with the reason."""
import torch


def f(gen, *shape, lo=0.1, hi=0.9, dtype=torch.float32):
    return torch.rand(*shape, generator=gen, dtype=torch.float64).mul(hi - lo).add(lo).to(dtype)


def i(gen, lo, hi, *shape, dtype=torch.int64):
    return torch.randint(lo, hi, shape, generator=gen, dtype=dtype)


def scalar(v):
    return torch.tensor([float(v)])


SPECS = {}


def spec(*names):
    def deco(fn):
        for n in names:
            SPECS[n] = fn
        return fn
    return deco


def simple(names, tensors, **attrs):
    """Register one spec for several names: ``tensors`` is a callable gen -> list."""
    for n in names.split():
        SPECS[n] = (lambda t, a: (lambda gen: (t(gen), a)))(tensors, attrs)


# ---- creation operators (no array inputs) ------------------------------------------------------------------------------
simple('_arange _npi_arange', lambda g: [], start=1, stop=7, step=2.0)
simple('_eye _npi_eye', lambda g: [], N=3, M=4, k=1)
simple('_full _npi_full', lambda g: [], shape=(2, 3), value=1.5)
simple('_linspace _npi_linspace', lambda g: [], start=0.0, stop=2.0, num=5)
simple('_npi_logspace', lambda g: [], start=0.0, stop=2.0, num=5)
simple('_npi_blackman _npi_hamming _npi_hanning', lambda g: [], M=6)
simple('_npi_identity', lambda g: [], shape=(3, 3))
simple('_npi_ones _ones _npi_zeros _zeros _zeros_without_dtype', lambda g: [], shape=(2, 3))
simple('_npi_tri', lambda g: [], N=3, M=4, k=0)
simple('_npi_tril_indices', lambda g: [], n=4, k=0, m=3)
simple('_random_uniform random_uniform uniform', lambda g: [], low=0.0, high=2.0, shape=(3, 4))
simple('_random_normal random_normal normal', lambda g: [], loc=0.0, scale=2.0, shape=(3, 4))
simple('_random_exponential random_exponential', lambda g: [], lam=2.0, shape=(3, 4))
simple('_random_gamma random_gamma', lambda g: [], alpha=2.0, beta=1.5, shape=(3, 4))
simple('_random_poisson random_poisson', lambda g: [], lam=3.0, shape=(3, 4))
simple('_random_negative_binomial random_negative_binomial', lambda g: [], k=3, p=0.4, shape=(3, 4))
simple('_random_binomial random_binomial', lambda g: [], n=5, p=0.4, shape=(3, 4))
simple('_random_randint random_randint', lambda g: [], low=0, high=9, shape=(3, 4))
simple('_npi_randint', lambda g: [], low=0, high=9, size=(3, 4))
simple('_sample_unique_zipfian', lambda g: [], range_max=50, shape=(2, 8))
simple('_npi_pareto _npi_powerd _npi_rayleigh _npi_weibull', lambda g: [f(g, 3, 4, lo=1.0, hi=2.0)])

# ---- shape manipulation --------------------------------------------------------------------------------------------------
simple('Reshape reshape', lambda g: [f(g, 3, 4)], shape=(4, 3))
simple('_np_reshape _npi_reshape _npx_reshape', lambda g: [f(g, 3, 4)], newshape=(2, 6))
simple('_npi_broadcast_to broadcast_to', lambda g: [f(g, 1, 4)], shape=(3, 4))
simple('_contrib_dynamic_reshape', lambda g: [f(g, 3, 4), torch.tensor([4, 3])])
simple('_npi_clip clip', lambda g: [f(g, 3, 4)], a_min=0.3, a_max=0.6)
simple('_npi_cross', lambda g: [f(g, 4, 3), f(g, 4, 3)])
simple('_npi_einsum', lambda g: [f(g, 3, 4), f(g, 4, 5)], subscripts='ij,jk->ik', num_args=2)
simple('_npi_digitize', lambda g: [f(g, 3, 4), torch.tensor([0.2, 0.4, 0.6, 0.8])])
simple('_npi_partition', lambda g: [f(g, 3, 6)], kth=2)
simple('_npi_tensorinv', lambda g: [torch.eye(6).reshape(2, 3, 6) + f(g, 2, 3, 6) * 0.1], ind=2)
simple('_npi_tensorsolve', lambda g: [torch.eye(6).reshape(2, 3, 6) + f(g, 2, 3, 6) * 0.1, f(g, 2, 3)])
simple('_npi_matrix_rank _npi_matrix_rank_none_tol', lambda g: [f(g, 4, 4)])
simple('_npi_cholesky _linalg_potrf linalg_potrf',
       lambda g: [(lambda a: a @ a.transpose(-1, -2) + 4 * torch.eye(4))(f(g, 4, 4))])
simple('_ravel_multi_index ravel_multi_index', lambda g: [torch.stack([i(g, 0, 3, 5), i(g, 0, 4, 5)])], shape=(3, 4))
simple('_unravel_index unravel_index', lambda g: [i(g, 0, 12, 5)], shape=(3, 4))
simple('scatter_nd _backward_gather_nd', lambda g: [f(g, 4), torch.tensor([[0, 1, 2, 0], [0, 1, 2, 3]])], shape=(3, 4))
simple('_scatter_set_nd', lambda g: [f(g, 3, 4), f(g, 4), torch.tensor([[0, 1, 2, 0], [0, 1, 2, 3]])], shape=(3, 4))
simple('_npx_index_add index_add', lambda g: [f(g, 3, 4), torch.tensor([[0, 2], [1, 3]]), f(g, 2)])
simple('_npx_index_update index_update', lambda g: [f(g, 3, 4), torch.tensor([[0, 2], [1, 3]]), f(g, 2)])
simple('im2col', lambda g: [f(g, 2, 3, 6, 6)], kernel=(3, 3), stride=(1, 1), pad=(1, 1))
simple('col2im', lambda g: [f(g, 2, 27, 36)], output_size=(6, 6), kernel=(3, 3), stride=(1, 1), pad=(1, 1))

# ---- integer scalar operators ----------------------------------------------------------------------------------------------
simple('_bitwise_and_scalar _bitwise_or_scalar _bitwise_xor_scalar _npi_bitwise_and_scalar _npi_bitwise_or_scalar '
       '_npi_bitwise_xor_scalar _rbitwise_and_scalar _rbitwise_or_scalar _rbitwise_xor_scalar _npi_rbitwise_and_scalar '
       '_npi_rbitwise_or_scalar _npi_rbitwise_xor_scalar _npi_gcd_scalar _npi_lcm_scalar _npi_rgcd_scalar _npi_rlcm_scalar',
       lambda g: [i(g, 1, 20, 3, 4)], scalar=6, is_int=True)
simple('_left_shift_scalar _right_shift_scalar _rleft_shift_scalar _rright_shift_scalar _npi_left_shift_scalar '
       '_npi_right_shift_scalar _npi_rleft_shift_scalar _npi_rright_shift_scalar _npi_bitwise_left_shift_scalar '
       '_npi_bitwise_right_shift_scalar _npi_rbitwise_left_shift_scalar _npi_rbitwise_right_shift_scalar',
       lambda g: [i(g, 1, 5, 3, 4)], scalar=2, is_int=True)

# ---- neural-network layers -----------------------------------------------------------------------------------------------
simple('Pooling Pooling_v1 _npx_pooling', lambda g: [f(g, 2, 3, 8, 8)], kernel=(2, 2), stride=(2, 2), pool_type='max')
simple('Deconvolution _npx_deconvolution', lambda g: [f(g, 2, 4, 5, 5), f(g, 4, 3, 3, 3)], kernel=(3, 3), num_filter=3,
       stride=(2, 2), pad=(1, 1), adj=(1, 1))
simple('GroupNorm _npx_group_norm', lambda g: [f(g, 2, 4, 5, 5), f(g, 4), f(g, 4)], num_groups=2)
simple('InstanceNorm _npx_instance_norm', lambda g: [f(g, 2, 3, 5, 5), f(g, 3), f(g, 3)])
simple('BilinearSampler', lambda g: [f(g, 2, 3, 6, 6), f(g, 2, 2, 4, 4, lo=-0.9, hi=0.9)])
simple('GridGenerator', lambda g: [f(g, 2, 6, lo=-0.5, hi=0.5)], transform_type='affine', target_shape=(4, 5))
simple('SpatialTransformer', lambda g: [f(g, 2, 3, 6, 6), f(g, 2, 6, lo=-0.5, hi=0.5)], target_shape=(4, 5),
       transform_type='affine', sampler_type='bilinear')
simple('CTCLoss _contrib_CTCLoss _contrib_ctc_loss ctc_loss _npx_ctc_loss',
       lambda g: [f(g, 6, 2, 5), torch.tensor([[1., 2., 0.], [3., 1., 2.]])])


def _rnn(gen):
    from mxnet_b200.ops.nn import rnn_param_size
    T, N, I, H = 4, 2, 3, 5
    return [f(gen, T, N, I), f(gen, rnn_param_size('lstm', 1, I, H), lo=-0.3, hi=0.3), f(gen, 1, N, H), f(gen, 1, N, H)], \
        dict(state_size=H, num_layers=1, mode='lstm', state_outputs=True)


SPECS['RNN'] = SPECS['_npx_rnn'] = _rnn


def _rois(gen, n=3):
    xy = f(gen, n, 2, lo=0.0, hi=3.0)
    wh = f(gen, n, 2, lo=2.0, hi=4.0)
    return torch.cat([i(gen, 0, 2, n, 1).float(), xy, xy + wh], 1)


simple('ROIPooling', lambda g: [f(g, 2, 3, 8, 8), _rois(g)], pooled_size=(2, 2), spatial_scale=1.0)
simple('ROIAlign _contrib_ROIAlign', lambda g: [f(g, 2, 3, 8, 8), _rois(g)], pooled_size=(2, 2), spatial_scale=1.0,
       sample_ratio=2)
simple('RROIAlign _contrib_RROIAlign',
       lambda g: [f(g, 2, 3, 8, 8), torch.cat([i(g, 0, 2, 3, 1).float(), f(g, 3, 2, lo=3.0, hi=5.0), f(g, 3, 2, lo=2.0, hi=4.0),
                                                f(g, 3, 1, lo=0.0, hi=45.0)], 1)], pooled_size=(2, 2), spatial_scale=1.0,
       sampling_ratio=2)
simple('PSROIPooling _contrib_PSROIPooling', lambda g: [f(g, 2, 8, 8, 8), _rois(g)], spatial_scale=1.0, output_dim=2,
       pooled_size=2, group_size=2)
simple('DeformablePSROIPooling _contrib_DeformablePSROIPooling', lambda g: [f(g, 2, 8, 8, 8), _rois(g)], spatial_scale=1.0,
       output_dim=2, group_size=2, pooled_size=2, no_trans=True)
simple('DeformableConvolution _contrib_DeformableConvolution',
       lambda g: [f(g, 2, 3, 6, 6), f(g, 2, 18, 6, 6, lo=-0.4, hi=0.4), f(g, 4, 3, 3, 3), f(g, 4)], kernel=(3, 3), pad=(1, 1),
       num_filter=4)
simple('ModulatedDeformableConvolution _contrib_ModulatedDeformableConvolution',
       lambda g: [f(g, 2, 3, 6, 6), f(g, 2, 18, 6, 6, lo=-0.4, hi=0.4), f(g, 2, 9, 6, 6), f(g, 4, 3, 3, 3), f(g, 4)],
       kernel=(3, 3), pad=(1, 1), num_filter=4)
simple('MultiBoxDetection _contrib_MultiBoxDetection',
       lambda g: [torch.softmax(f(g, 2, 3, 4), 1), f(g, 2, 16, lo=-0.2, hi=0.2),
                  torch.cat([f(g, 1, 4, 2, lo=0.0, hi=0.4), f(g, 1, 4, 2, lo=0.5, hi=0.9)], 2)])
simple('Proposal _contrib_Proposal MultiProposal _contrib_MultiProposal',
       lambda g: [f(g, 1, 6, 4, 4), f(g, 1, 12, 4, 4, lo=-0.2, hi=0.2), torch.tensor([[64., 64., 1.]])], scales=(4.0,),
       ratios=(0.5, 1.0, 2.0), feature_stride=16, rpn_pre_nms_top_n=20, rpn_post_nms_top_n=5, rpn_min_size=2)
simple('_contrib_box_encode box_encode',
       lambda g: [torch.tensor([[1., 0., 1.]]), torch.tensor([[0, 1, 0]]), torch.cat([f(g, 1, 3, 2, hi=0.4), f(g, 1, 3, 2, lo=0.5)], 2),
                  torch.cat([f(g, 1, 2, 2, hi=0.4), f(g, 1, 2, 2, lo=0.5)], 2), torch.zeros(4), torch.ones(4)])
simple('_contrib_mrcnn_mask_target mrcnn_mask_target',
       lambda g: [torch.cat([f(g, 1, 3, 2, lo=0.0, hi=3.0), f(g, 1, 3, 2, lo=5.0, hi=7.0)], 2), (f(g, 1, 2, 8, 8) > 0.5).float(),
                  torch.tensor([[0., 1., 0.]]), torch.tensor([[1., 2., 0.]])], num_rois=3, num_classes=3, mask_size=(4, 4))
simple('_contrib_count_sketch count_sketch', lambda g: [f(g, 3, 8), i(g, 0, 5, 1, 8).float(), (i(g, 0, 2, 1, 8) * 2 - 1).float()],
       out_dim=5)
simple('_contrib_hawkesll hawkesll',
       lambda g: [f(g, 2, 3), f(g, 3), f(g, 3, lo=1.0, hi=2.0), f(g, 2, 3), f(g, 2, 5), i(g, 0, 3, 2, 5).int(),
                  torch.tensor([5., 4.]), torch.tensor([6., 6.])])

# ---- attention -------------------------------------------------------------------------------------------------------------
simple('_contrib_interleaved_matmul_selfatt_qk interleaved_matmul_selfatt_qk', lambda g: [f(g, 5, 2, 2 * 3 * 4)], heads=2)
simple('_contrib_interleaved_matmul_selfatt_valatt interleaved_matmul_selfatt_valatt',
       lambda g: [f(g, 5, 2, 2 * 3 * 4), f(g, 4, 5, 5)], heads=2)
simple('_contrib_interleaved_matmul_encdec_qk interleaved_matmul_encdec_qk', lambda g: [f(g, 5, 2, 8), f(g, 6, 2, 16)], heads=2)
simple('_contrib_interleaved_matmul_encdec_valatt interleaved_matmul_encdec_valatt',
       lambda g: [f(g, 6, 2, 16), f(g, 4, 5, 6)], heads=2)
simple('_contrib_fused_self_attention fused_self_attention _npx_fused_self_attention', lambda g: [f(g, 2, 5, 3 * 8)], heads=2)
simple('_contrib_sldwin_atten_score', lambda g: [f(g, 2, 6, 2, 4), f(g, 2, 6, 2, 4), torch.ones(2, dtype=torch.int32)], w=2,
       symmetric=True)
simple('_contrib_sldwin_atten_mask_like',
       lambda g: [f(g, 2, 6, 2, 5), torch.ones(2, dtype=torch.int32), torch.tensor([6, 4], dtype=torch.int32)], w=2, symmetric=True)
simple('_contrib_sldwin_atten_context', lambda g: [f(g, 2, 6, 2, 5), f(g, 2, 6, 2, 4), torch.ones(2, dtype=torch.int32)], w=2,
       symmetric=True)

# ---- image operators ---------------------------------------------------------------------------------------------------------
simple('_image_adjust_lighting _npx__image_adjust_lighting', lambda g: [f(g, 6, 5, 3)], alpha=(0.1, 0.2, 0.3))
simple('_image_random_contrast _npx__image_random_contrast _image_random_saturation _npx__image_random_saturation '
       '_image_random_hue _npx__image_random_hue', lambda g: [f(g, 6, 5, 3)], min_factor=0.8, max_factor=1.2)
simple('_image_random_lighting _npx__image_random_lighting', lambda g: [f(g, 6, 5, 3)], alpha_std=0.05)
simple('_image_resize _npx__image_resize', lambda g: [f(g, 6, 5, 3)], size=(4, 3))
simple('_cvcopyMakeBorder', lambda g: [(f(g, 6, 5, 3) * 255).to(torch.uint8)], top=1, bot=2, left=1, right=0)

# ---- quantisation ------------------------------------------------------------------------------------------------------------
_q8 = lambda g, *s: i(g, -100, 100, *s).to(torch.int8)                               # noqa: E731
_rng = lambda v: [torch.tensor([-float(v)]), torch.tensor([float(v)])]              # noqa: E731
simple('_contrib_quantize quantize', lambda g: [f(g, 3, 4, lo=-1.0, hi=1.0)] + _rng(1.0), out_type='int8')
simple('_contrib_dequantize dequantize', lambda g: [_q8(g, 3, 4)] + _rng(1.0))
simple('_contrib_requantize requantize', lambda g: [i(g, -100000, 100000, 3, 4).int()] + _rng(50.0))
simple('_contrib_quantized_fully_connected', lambda g: [_q8(g, 3, 16), _q8(g, 5, 16), _q8(g, 5)] + _rng(1.0) + _rng(0.5) + _rng(2.0),
       num_hidden=5)
simple('_contrib_quantized_conv', lambda g: [_q8(g, 2, 3, 6, 6), _q8(g, 4, 3, 3, 3), _q8(g, 4)] + _rng(1.0) + _rng(0.5) + _rng(2.0),
       kernel=(3, 3), num_filter=4, pad=(1, 1))
simple('_contrib_quantized_pooling', lambda g: [_q8(g, 2, 3, 6, 6)] + _rng(1.0), kernel=(2, 2), stride=(2, 2), pool_type='max')
simple('_contrib_quantized_reshape', lambda g: [_q8(g, 3, 4)] + _rng(1.0), shape=(4, 3))
simple('_npx_quantized_reshape', lambda g: [_q8(g, 3, 4)] + _rng(1.0), newshape=(4, 3))
simple('_contrib_quantized_elemwise_add _contrib_quantized_elemwise_mul _contrib_quantized_npi_add',
       lambda g: [_q8(g, 3, 4), _q8(g, 3, 4)] + _rng(1.0) + _rng(2.0))
simple('_contrib_quantized_batch_norm _contrib_quantized_batch_norm_relu',
       lambda g: [_q8(g, 2, 3, 4, 4), f(g, 3), f(g, 3), f(g, 3), f(g, 3, lo=0.5, hi=1.5)] + _rng(1.0))
simple('_contrib_quantized_concat', lambda g: [_q8(g, 2, 3), _q8(g, 2, 4)] + _rng(1.0) + _rng(2.0), num_args=2, dim=1)
simple('_contrib_intgemm_prepare_data intgemm_prepare_data', lambda g: [f(g, 4, 64, lo=-1.0, hi=1.0), torch.tensor([1.0])])
simple('_contrib_intgemm_prepare_weight intgemm_prepare_weight', lambda g: [f(g, 8, 64, lo=-1.0, hi=1.0), torch.tensor([1.0])])


def _quantized_rnn(gen):
    tensors, attrs = _rnn(gen)
    return tensors + [torch.tensor([64.0]), torch.tensor([0.0])], attrs


SPECS['_contrib_quantized_rnn'] = SPECS['quantized_rnn'] = _quantized_rnn

# ---- multi-tensor optimizer updates ---------------------------------------------------------------------------------------------
_w = lambda g: f(g, 3, 4, lo=-0.5, hi=0.5)                                            # noqa: E731
_v = lambda g: f(g, 3, 4, lo=0.01, hi=0.1)                                            # noqa: E731
simple('multi_sgd_update', lambda g: [_w(g), _w(g), _w(g), _w(g)], lrs=(0.1, 0.2), wds=(0.0, 0.01), num_weights=2)
simple('multi_sgd_mom_update', lambda g: [_w(g), _w(g), _w(g)] * 2, lrs=(0.1, 0.2), wds=(0.0, 0.01), momentum=0.9, num_weights=2)
simple('multi_mp_sgd_update', lambda g: [_w(g).half(), _w(g).half(), _w(g)] * 2, lrs=(0.1, 0.2), wds=(0.0, 0.01), num_weights=2)
simple('multi_mp_sgd_mom_update', lambda g: [_w(g).half(), _w(g).half(), _w(g), _w(g)] * 2, lrs=(0.1, 0.2), wds=(0.0, 0.01),
       momentum=0.9, num_weights=2)
_lw = lambda g: [torch.tensor([0.1, 0.2]), torch.tensor([0.0, 0.01])]                # noqa: E731
simple('preloaded_multi_sgd_update', lambda g: [_w(g), _w(g), _w(g), _w(g)] + _lw(g), num_weights=2)
simple('preloaded_multi_sgd_mom_update', lambda g: [_w(g), _w(g), _w(g)] * 2 + _lw(g), momentum=0.9, num_weights=2)
simple('preloaded_multi_mp_sgd_update', lambda g: [_w(g).half(), _w(g).half(), _w(g)] * 2 + _lw(g), num_weights=2)
simple('preloaded_multi_mp_sgd_mom_update', lambda g: [_w(g).half(), _w(g).half(), _w(g), _w(g)] * 2 + _lw(g), momentum=0.9,
       num_weights=2)
_adam = dict(lrs=(0.01, 0.02), wds=(0.0, 0.01), etas=(1.0, 1.0), num_weights=2)
simple('_multi_adamw_update _contrib_multi_adamw_update', lambda g: [_w(g), _w(g), _w(g), _v(g)] * 2 + [torch.tensor([1.0])], **_adam)
simple('_multi_mp_adamw_update _contrib_multi_mp_adamw_update',
       lambda g: [_w(g).half(), _w(g).half(), _w(g), _v(g), _w(g)] * 2 + [torch.tensor([1.0])], **_adam)
simple('_multi_adabelief_update _contrib_multi_adabelief_update',
       lambda g: [_w(g), _w(g), _w(g), _v(g)] * 2 + [torch.tensor([1.0])], **_adam)
simple('_multi_mp_adabelief_update _contrib_multi_mp_adabelief_update',
       lambda g: [_w(g).half(), _w(g).half(), _w(g), _v(g), _w(g)] * 2 + [torch.tensor([1.0])], **_adam)
_lamb = dict(learning_rates=(0.01, 0.02), wds=(0.0, 0.01), step_count=(1, 3), num_tensors=2)
simple('_multi_lamb_update _multi_lans_update', lambda g: [_w(g), _w(g), _w(g), _v(g)] * 2, **_lamb)
simple('_multi_mp_lamb_update _multi_mp_lans_update', lambda g: [_w(g).half(), _w(g).half(), _w(g), _v(g), _w(g)] * 2, **_lamb)
simple('lamb_update_phase2', lambda g: [_w(g), _w(g), torch.tensor([1.5]), torch.tensor([0.7])], lr=0.01)
simple('mp_lamb_update_phase2', lambda g: [_w(g).half(), _w(g), torch.tensor([1.5]), torch.tensor([0.7]), _w(g)], lr=0.01)

# ---- names the sweep leaves out ----------------------------------------------------------------------------------------------
EXCLUDED = {
    '_foreach': 'control-flow node: its body is a sub-graph attribute (tested in test_symbol.py / test_contrib_misc.py)',
    '_while_loop': 'control-flow node with sub-graph attributes',
    '_cond': 'control-flow node with sub-graph attributes',
    '_FusedOp': 'created by the pointwise fusion pass only (tests/test_fusion.py)',
    'Custom': 'dispatches to a user-registered Python operator (tests/test_misc_api.py)',
    '_cvimread': 'reads an image file (tests/test_io.py)',
    '_cvimdecode': 'decodes an encoded image buffer (tests/test_io.py)',
    '_contrib_dgl_graph_compact': 'takes CSR graph containers, not dense arrays (tests/test_contrib_misc.py)',
}

# operators whose outputs draw from a random generator: determinism, NumPy and gradient checks do not apply
RANDOM_PATTERN = (r'random|sample|_npi_(normal|uniform|gamma|exponential|binomial|bernoulli|choice|multinomial|gumbel|logistic|'
                  r'laplace|pareto|powerd|rayleigh|weibull|randint|shuffle|permutation|dirichlet|beta|chisquare|f$|standard)|'
                  r'[Dd]ropout|shuffle|^normal$|^uniform$|_rnn_param_concat$')

# not differentiable at generic points, or the finite difference crosses a discontinuity of the operator
_BY_DESIGN = 'the backward pass is defined by the operator (a loss gradient or a straight-through estimate), not the derivative of its forward'
_SYMMETRIC = 'reads its input as a symmetric / triangular matrix: an element-wise perturbation leaves its domain'
_INDEX = 'an input holds indices or box corners: the output is piecewise constant or discontinuous in it'
NO_GRADCHECK = {
    'LinearRegressionOutput': _BY_DESIGN, 'LogisticRegressionOutput': _BY_DESIGN, 'MAERegressionOutput': _BY_DESIGN,
    'SoftmaxOutput': _BY_DESIGN, 'Softmax': _BY_DESIGN, 'SVMOutput': _BY_DESIGN, '_contrib_round_ste': _BY_DESIGN,
    '_contrib_sign_ste': _BY_DESIGN, 'MakeLoss': _BY_DESIGN, 'make_loss': _BY_DESIGN, 'BlockGrad': _BY_DESIGN,
    '_contrib_gradientmultiplier': _BY_DESIGN, 'IdentityAttachKLSparseReg': _BY_DESIGN,
    '_linalg_potrf': _SYMMETRIC, '_npi_cholesky': _SYMMETRIC, '_linalg_potri': _SYMMETRIC, '_linalg_syevd': _SYMMETRIC,
    '_npi_eigh': _SYMMETRIC, '_npi_eigvalsh': _SYMMETRIC, '_linalg_trmm': _SYMMETRIC, '_linalg_trsm': _SYMMETRIC,
    '_linalg_syrk': _SYMMETRIC, '_linalg_inverse': None, '_npi_eig': 'complex eigenvectors are defined up to a phase',
    '_npi_eigvals': 'complex eigenvalues', '_contrib_quantize': 'rounds to integers', '_contrib_quantize_v2': 'rounds to integers',
    '_contrib_quantize_asym': 'rounds to integers', '_contrib_requantize': 'rounds to integers',
    '_contrib_index_copy': _INDEX, '_contrib_count_sketch': _INDEX, '_contrib_mrcnn_mask_target': _INDEX,
    '_sparse_retain': _INDEX, '_sparse_retain_dense': _INDEX, '_contrib_box_encode': _INDEX, '_contrib_hawkesll': _INDEX,
}
NO_GRADCHECK = {k: v for k, v in NO_GRADCHECK.items() if v}

# operators of which only some inputs are differentiable (positions): the others are boxes, indices or counts
GRAD_INPUTS = {
    'ROIPooling': (0,), 'ROIAlign': (0,), 'RROIAlign': (0,), 'PSROIPooling': (0,), 'DeformablePSROIPooling': (0,),
    'MultiBoxDetection': (), 'Proposal': (), 'MultiProposal': (), 'CTCLoss': (0,),
    '_contrib_sldwin_atten_score': (0, 1), '_contrib_sldwin_atten_context': (0, 1), '_contrib_sldwin_atten_mask_like': (0,),
}

# outputs defined up to a sign, a phase or an order (eigenvectors, singular vectors): two libraries may differ
NO_DEVICE_COMPARE = {'_npi_eig', '_npi_eigh', '_npi_svd', '_linalg_syevd', '_linalg_gelqf', '_npi_qr', '_npi_eigvals',
                     '_linalg_svd', '_npi_pinv', '_npi_lstsq'}

# `_npi_<name>` whose argument convention differs from `numpy.<name>` (attributes instead of arrays, other defaults)
NO_NUMPY = {'_npi_flip', '_npi_insert', '_npi_interp', '_npi_delete', '_npi_pad', '_npi_around', '_npi_std', '_npi_var'}

simple('MultiBoxTarget _contrib_MultiBoxTarget',
       lambda g: [torch.cat([f(g, 1, 6, 2, lo=0.0, hi=0.4), f(g, 1, 6, 2, lo=0.5, hi=0.9)], 2),
                  torch.tensor([[[0., 0.1, 0.1, 0.6, 0.7], [-1., 0., 0., 0., 0.]], [[1., 0.2, 0.3, 0.8, 0.9], [0., 0.05, 0.1, 0.5, 0.6]]]),
                  f(g, 2, 3, 6)])
simple('_image_random_flip_top_bottom _npx__image_random_flip_top_bottom _image_random_flip_left_right '
       '_npx__image_random_flip_left_right _image_flip_top_bottom _image_flip_left_right', lambda g: [f(g, 6, 5, 3)])
simple('_contrib_calibrate_entropy calibrate_entropy',
       lambda g: [torch.histc(torch.randn(4000, generator=g), 401, -4, 4), torch.linspace(-4, 4, 402)], num_quantized_bins=31)
simple('_contrib_index_copy index_copy', lambda g: [f(g, 5, 4), torch.tensor([3, 0, 4]), f(g, 3, 4)])
