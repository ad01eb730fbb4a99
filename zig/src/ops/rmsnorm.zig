// y = x * rsqrt(mean_j x^2 + eps) * gain over the last axis of a rank-2 tensor.  The reverse needs scratch for
// the per-CTA partial sums of the gain gradient: it comes from the stream's grow-only scratch
// (StreamEntry.get_scratch, src/core/utils.zig:20-36), sized by mpRmsnormReverseScratchBytes.
const std = @import("std");
const core = @import("core");
const OpDatum = core.OpDatum;
const Tensor = core.Tensor;
const Graph = core.Graph;
const C = @import("../core/cimport.zig").C;

pub fn forward(x: Tensor, gain: Tensor, eps: f64) Tensor {
    return forward_impl(x.ptr, x, gain, eps);
}

pub fn forward_impl(graph: *Graph, x: Tensor, gain: Tensor, eps: f64) Tensor {
    const xs = x.sizes();
    std.debug.assert(xs.len == 2 and gain.len() == xs[1]);

    const y = graph.tensor(.{ .class = .hid, .dtype = x.dtype(), .sizes = xs });

    // rstd is not kept: the reverse recomputes it from x (one extra reduction that is free in a memory-bound kernel)
    core.invoke(core.kernels.rmsnorm_ij_j, core.dkey(y), .{
        x.data_ptr(),
        gain.data_ptr(),
        eps,
        y.data_ptr(),
        @as(?*anyopaque, null),
        xs[0],
        xs[1],
        y.context(),
    });

    if (graph.mode == .train) {
        core.attach_op(@This(), y, &.{
            OpDatum{ .tensor = x },
            OpDatum{ .tensor = gain },
            OpDatum{ .scalar = eps },
            OpDatum{ .tensor = y },
        });
    }
    return y;
}

// g_x += r (g_y o gain) - x r^3 mean_j(g_y o gain o x),  g_gain += sum_i g_y o x r_i
pub fn reverse(args: []const OpDatum) void {
    const x = args[0].tensor;
    const gain = args[1].tensor;
    const eps = args[2].scalar;
    const y = args[3].tensor;
    const xs = x.sizes();

    core.enable_gradient(x);
    core.enable_gradient(gain);

    const bytes = C.mpRmsnormReverseScratchBytes(xs[0], xs[1], y.context());
    const scratch = y.ptr.stream.get_scratch(.r64, (bytes + 7) / 8);

    core.invoke(core.kernels.rmsnorm_ij_j_reverse, core.dkey(y), .{
        x.data_ptr(),
        gain.data_ptr(),
        @as(?*const anyopaque, null),
        y.grad_ptr(),
        eps,
        x.grad_ptr(),
        gain.grad_ptr(),
        1.0,
        scratch,
        xs[0],
        xs[1],
        y.context(),
    });
}

pub fn derive(_: []const OpDatum, _: Tensor) ?OpDatum {
    return null;
}
