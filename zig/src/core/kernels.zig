// Replaces the generated src/core/kernels.zig (file_gen.zig:298-328).  One array per launcher, ordered like the
// dtype key of src/core/scalar.zig:35-40 (r16, r32, r64), for core.invoke (src/core/root.zig:36-43).
// The first twenty names are the reference's own (src/cuda/kernel_decls.h:11-436); the rest are the additive launchers.

const decls = @import("cimport.zig").C;

fn dispatch_array(comptime _: anytype, comptime tuple: anytype) [tuple.len]@TypeOf(tuple[0]) {
    return tuple;
}

pub const reduce_ij_i = dispatch_array(opaque {}, .{
    decls.launch_reduce_ij_i_r16,
    decls.launch_reduce_ij_i_r32,
    decls.launch_reduce_ij_i_r64,
});

pub const reduce_ij_j = dispatch_array(opaque {}, .{
    decls.launch_reduce_ij_j_r16,
    decls.launch_reduce_ij_j_r32,
    decls.launch_reduce_ij_j_r64,
});

pub const broadcast_i_ij = dispatch_array(opaque {}, .{
    decls.launch_broadcast_i_ij_r16,
    decls.launch_broadcast_i_ij_r32,
    decls.launch_broadcast_i_ij_r64,
});

pub const broadcast_j_ij = dispatch_array(opaque {}, .{
    decls.launch_broadcast_j_ij_r16,
    decls.launch_broadcast_j_ij_r32,
    decls.launch_broadcast_j_ij_r64,
});

pub const dilate_reverse = dispatch_array(opaque {}, .{
    decls.launch_dilate_reverse_r16,
    decls.launch_dilate_reverse_r32,
    decls.launch_dilate_reverse_r64,
});

pub const subtraction = dispatch_array(opaque {}, .{
    decls.launch_subtraction_r16,
    decls.launch_subtraction_r32,
    decls.launch_subtraction_r64,
});

pub const relu_reverse = dispatch_array(opaque {}, .{
    decls.launch_relu_reverse_r16,
    decls.launch_relu_reverse_r32,
    decls.launch_relu_reverse_r64,
});

pub const dilate = dispatch_array(opaque {}, .{
    decls.launch_dilate_r16,
    decls.launch_dilate_r32,
    decls.launch_dilate_r64,
});

pub const translate = dispatch_array(opaque {}, .{
    decls.launch_translate_r16,
    decls.launch_translate_r32,
    decls.launch_translate_r64,
});

pub const permutate_ij_ji = dispatch_array(opaque {}, .{
    decls.launch_permutate_ij_ji_r16,
    decls.launch_permutate_ij_ji_r32,
    decls.launch_permutate_ij_ji_r64,
});

pub const negate = dispatch_array(opaque {}, .{
    decls.launch_negate_r16,
    decls.launch_negate_r32,
    decls.launch_negate_r64,
});

pub const hadamard_reverse = dispatch_array(opaque {}, .{
    decls.launch_hadamard_reverse_r16,
    decls.launch_hadamard_reverse_r32,
    decls.launch_hadamard_reverse_r64,
});

pub const inner_product_ij_jk_ik = dispatch_array(opaque {}, .{
    decls.launch_inner_product_ij_jk_ik_r16,
    decls.launch_inner_product_ij_jk_ik_r32,
    decls.launch_inner_product_ij_jk_ik_r64,
});

pub const hadamard = dispatch_array(opaque {}, .{
    decls.launch_hadamard_r16,
    decls.launch_hadamard_r32,
    decls.launch_hadamard_r64,
});

pub const fill = dispatch_array(opaque {}, .{
    decls.launch_fill_r16,
    decls.launch_fill_r32,
    decls.launch_fill_r64,
});

pub const relu = dispatch_array(opaque {}, .{
    decls.launch_relu_r16,
    decls.launch_relu_r32,
    decls.launch_relu_r64,
});

pub const addition = dispatch_array(opaque {}, .{
    decls.launch_addition_r16,
    decls.launch_addition_r32,
    decls.launch_addition_r64,
});

pub const copy = dispatch_array(opaque {}, .{
    decls.launch_copy_r16,
    decls.launch_copy_r32,
    decls.launch_copy_r64,
});

pub const sequence = dispatch_array(opaque {}, .{
    decls.launch_sequence_r16,
    decls.launch_sequence_r32,
    decls.launch_sequence_r64,
});

pub const stepwise = dispatch_array(opaque {}, .{
    decls.launch_stepwise_r16,
    decls.launch_stepwise_r32,
    decls.launch_stepwise_r64,
});

pub const selu = dispatch_array(opaque {}, .{
    decls.launch_selu_r16,
    decls.launch_selu_r32,
    decls.launch_selu_r64,
});

pub const selu_reverse = dispatch_array(opaque {}, .{
    decls.launch_selu_reverse_r16,
    decls.launch_selu_reverse_r32,
    decls.launch_selu_reverse_r64,
});

pub const softmax_ij_j = dispatch_array(opaque {}, .{
    decls.launch_softmax_ij_j_r16,
    decls.launch_softmax_ij_j_r32,
    decls.launch_softmax_ij_j_r64,
});

pub const softmax_ij_j_reverse = dispatch_array(opaque {}, .{
    decls.launch_softmax_ij_j_reverse_r16,
    decls.launch_softmax_ij_j_reverse_r32,
    decls.launch_softmax_ij_j_reverse_r64,
});

pub const rmsnorm_ij_j = dispatch_array(opaque {}, .{
    decls.launch_rmsnorm_ij_j_r16,
    decls.launch_rmsnorm_ij_j_r32,
    decls.launch_rmsnorm_ij_j_r64,
});

pub const rmsnorm_ij_j_reverse = dispatch_array(opaque {}, .{
    decls.launch_rmsnorm_ij_j_reverse_r16,
    decls.launch_rmsnorm_ij_j_reverse_r32,
    decls.launch_rmsnorm_ij_j_reverse_r64,
});

pub const sgd = dispatch_array(opaque {}, .{
    decls.launch_sgd_r16,
    decls.launch_sgd_r32,
    decls.launch_sgd_r64,
});

pub const adam = dispatch_array(opaque {}, .{
    decls.launch_adam_r16,
    decls.launch_adam_r32,
    decls.launch_adam_r64,
});

pub const inner_product_ij_kj_ik = dispatch_array(opaque {}, .{
    decls.launch_inner_product_ij_kj_ik_r16,
    decls.launch_inner_product_ij_kj_ik_r32,
    decls.launch_inner_product_ij_kj_ik_r64,
});

pub const inner_product_ji_jk_ik = dispatch_array(opaque {}, .{
    decls.launch_inner_product_ji_jk_ik_r16,
    decls.launch_inner_product_ji_jk_ik_r32,
    decls.launch_inner_product_ji_jk_ik_r64,
});

pub const linear_ij_jk_ik = dispatch_array(opaque {}, .{
    decls.launch_linear_ij_jk_ik_r16,
    decls.launch_linear_ij_jk_ik_r32,
    decls.launch_linear_ij_jk_ik_r64,
});

pub const ssd_scan = dispatch_array(opaque {}, .{
    decls.launch_ssd_scan_r16,
    decls.launch_ssd_scan_r32,
    decls.launch_ssd_scan_r64,
});

pub const ssd_scan_reverse = dispatch_array(opaque {}, .{
    decls.launch_ssd_scan_reverse_r16,
    decls.launch_ssd_scan_reverse_r32,
    decls.launch_ssd_scan_reverse_r64,
});

pub const embedding = dispatch_array(opaque {}, .{
    decls.launch_embedding_r16,
    decls.launch_embedding_r32,
    decls.launch_embedding_r64,
});

pub const embedding_reverse = dispatch_array(opaque {}, .{
    decls.launch_embedding_reverse_r16,
    decls.launch_embedding_reverse_r32,
    decls.launch_embedding_reverse_r64,
});

pub const causal_conv1d_silu = dispatch_array(opaque {}, .{
    decls.launch_causal_conv1d_silu_r16,
    decls.launch_causal_conv1d_silu_r32,
    decls.launch_causal_conv1d_silu_r64,
});

pub const causal_conv1d_silu_reverse = dispatch_array(opaque {}, .{
    decls.launch_causal_conv1d_silu_reverse_r16,
    decls.launch_causal_conv1d_silu_reverse_r32,
    decls.launch_causal_conv1d_silu_reverse_r64,
});

pub const causal_conv1d_silu_segments = dispatch_array(opaque {}, .{
    decls.launch_causal_conv1d_silu_segments_r16,
    decls.launch_causal_conv1d_silu_segments_r32,
    decls.launch_causal_conv1d_silu_segments_r64,
});

pub const causal_conv1d_silu_segments_reverse = dispatch_array(opaque {}, .{
    decls.launch_causal_conv1d_silu_segments_reverse_r16,
    decls.launch_causal_conv1d_silu_segments_reverse_r32,
    decls.launch_causal_conv1d_silu_segments_reverse_r64,
});

pub const softplus_bias = dispatch_array(opaque {}, .{
    decls.launch_softplus_bias_r16,
    decls.launch_softplus_bias_r32,
    decls.launch_softplus_bias_r64,
});

pub const softplus_bias_reverse = dispatch_array(opaque {}, .{
    decls.launch_softplus_bias_reverse_r16,
    decls.launch_softplus_bias_reverse_r32,
    decls.launch_softplus_bias_reverse_r64,
});

pub const ssd_gate = dispatch_array(opaque {}, .{
    decls.launch_ssd_gate_r16,
    decls.launch_ssd_gate_r32,
    decls.launch_ssd_gate_r64,
});

pub const ssd_gate_reverse = dispatch_array(opaque {}, .{
    decls.launch_ssd_gate_reverse_r16,
    decls.launch_ssd_gate_reverse_r32,
    decls.launch_ssd_gate_reverse_r64,
});

pub const head_scale_accumulate = dispatch_array(opaque {}, .{
    decls.launch_head_scale_accumulate_r16,
    decls.launch_head_scale_accumulate_r32,
    decls.launch_head_scale_accumulate_r64,
});

pub const cross_entropy = dispatch_array(opaque {}, .{
    decls.launch_cross_entropy_r16,
    decls.launch_cross_entropy_r32,
    decls.launch_cross_entropy_r64,
});

pub const neg_exp = dispatch_array(opaque {}, .{
    decls.launch_neg_exp_r16,
    decls.launch_neg_exp_r32,
    decls.launch_neg_exp_r64,
});

pub const mse_loss_i_i = dispatch_array(opaque {}, .{
    decls.launch_mse_loss_i_i_r16,
    decls.launch_mse_loss_i_i_r32,
    decls.launch_mse_loss_i_i_r64,
});

pub const bce_loss_i_i = dispatch_array(opaque {}, .{
    decls.launch_bce_loss_i_i_r16,
    decls.launch_bce_loss_i_i_r32,
    decls.launch_bce_loss_i_i_r64,
});

pub const momentum = dispatch_array(opaque {}, .{
    decls.launch_momentum_r16,
    decls.launch_momentum_r32,
    decls.launch_momentum_r64,
});

pub const permutate = dispatch_array(opaque {}, .{
    decls.launch_permutate_r16,
    decls.launch_permutate_r32,
    decls.launch_permutate_r64,
});

pub const inner_product_bij_bjk_bik = dispatch_array(opaque {}, .{
    decls.launch_inner_product_bij_bjk_bik_r16,
    decls.launch_inner_product_bij_bjk_bik_r32,
    decls.launch_inner_product_bij_bjk_bik_r64,
});

pub const inner_product_bij_bkj_bik = dispatch_array(opaque {}, .{
    decls.launch_inner_product_bij_bkj_bik_r16,
    decls.launch_inner_product_bij_bkj_bik_r32,
    decls.launch_inner_product_bij_bkj_bik_r64,
});

pub const inner_product_bji_bjk_bik = dispatch_array(opaque {}, .{
    decls.launch_inner_product_bji_bjk_bik_r16,
    decls.launch_inner_product_bji_bjk_bik_r32,
    decls.launch_inner_product_bji_bjk_bik_r64,
});

pub const linear_ij_jk_ik_ik = dispatch_array(opaque {}, .{
    decls.launch_linear_ij_jk_ik_ik_r16,
    decls.launch_linear_ij_jk_ik_ik_r32,
    decls.launch_linear_ij_jk_ik_ik_r64,
});

pub const ssd_gate_rmsnorm = dispatch_array(opaque {}, .{
    decls.launch_ssd_gate_rmsnorm_r16,
    decls.launch_ssd_gate_rmsnorm_r32,
    decls.launch_ssd_gate_rmsnorm_r64,
});

pub const ssd_gate_rmsnorm_reverse = dispatch_array(opaque {}, .{
    decls.launch_ssd_gate_rmsnorm_reverse_r16,
    decls.launch_ssd_gate_rmsnorm_reverse_r32,
    decls.launch_ssd_gate_rmsnorm_reverse_r64,
});

pub const causal_conv1d_silu_segments_reverse_skip = dispatch_array(opaque {}, .{
    decls.launch_causal_conv1d_silu_segments_reverse_skip_r16,
    decls.launch_causal_conv1d_silu_segments_reverse_skip_r32,
    decls.launch_causal_conv1d_silu_segments_reverse_skip_r64,
});

pub const ssd_scan_raw = dispatch_array(opaque {}, .{
    decls.launch_ssd_scan_raw_r16,
    decls.launch_ssd_scan_raw_r32,
    decls.launch_ssd_scan_raw_r64,
});

pub const ssd_scan_reverse_raw = dispatch_array(opaque {}, .{
    decls.launch_ssd_scan_reverse_raw_r16,
    decls.launch_ssd_scan_reverse_raw_r32,
    decls.launch_ssd_scan_reverse_raw_r64,
});
