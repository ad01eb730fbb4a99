// Row-wise softmax over the last axis of a rank-2 tensor ("ij|j", src/ops/expression_parsing.zig:319-340;
// intended use src/loss/loss.zig:204,226).
const std = @import("std");
const core = @import("core");
const OpDatum = core.OpDatum;
const Tensor = core.Tensor;
const Graph = core.Graph;

pub fn forward(x: Tensor) Tensor {
    return forward_impl(x.ptr, x);
}

pub fn forward_impl(graph: *Graph, x: Tensor) Tensor {
    const xs = x.sizes();
    std.debug.assert(xs.len == 2);

    const y = graph.tensor(.{ .class = .hid, .dtype = x.dtype(), .sizes = xs });

    core.invoke(core.kernels.softmax_ij_j, core.dkey(y), .{
        x.data_ptr(),
        y.data_ptr(),
        xs[0],
        xs[1],
        y.context(),
    });

    if (graph.mode == .train) {
        core.attach_op(@This(), y, &.{
            OpDatum{ .tensor = x },
            OpDatum{ .tensor = y },
        });
    }
    return y;
}

// g_x += y o (g_y - sum_j g_y o y)
pub fn reverse(args: []const OpDatum) void {
    const x = args[0].tensor;
    const y = args[1].tensor;
    const ys = y.sizes();

    core.enable_gradient(x);

    core.invoke(core.kernels.softmax_ij_j_reverse, core.dkey(y), .{
        y.data_ptr(),
        y.grad_ptr(),
        x.grad_ptr(),
        1.0,
        ys[0],
        ys[1],
        y.context(),
    });
}

pub fn derive(_: []const OpDatum, _: Tensor) ?OpDatum {
    return null; // a row reduction has no element-wise derivative
}
