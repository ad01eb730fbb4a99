// y = selu(x) = lambda * (x > 0 ? x : alpha * (exp(x) - 1)), named by README.md:97; modelled on src/ops/relu.zig.
const std = @import("std");
const core = @import("core");
const OpDatum = core.OpDatum;
const Tensor = core.Tensor;
const Graph = core.Graph;

pub fn forward(x: Tensor) Tensor {
    return forward_impl(x.ptr, x);
}

pub fn forward_impl(graph: *Graph, x: Tensor) Tensor {
    const z = graph.tensor(.{
        .class = .hid,
        .dtype = x.dtype(),
        .sizes = x.sizes(),
    });

    core.invoke(core.kernels.selu, core.dkey(z), .{
        x.data_ptr(),
        z.data_ptr(),
        z.len(),
        z.context(),
    });

    if (graph.mode == .train) {
        core.attach_op(@This(), z, &.{
            OpDatum{ .tensor = x },
            OpDatum{ .tensor = z },
        });
    }
    return z;
}

// g_x += g_z * lambda * (x > 0 ? 1 : alpha * exp(x))
pub fn reverse(args: []const OpDatum) void {
    const x = args[0].tensor;
    const z = args[1].tensor;

    core.enable_gradient(x);

    core.invoke(core.kernels.selu_reverse, core.dkey(z), .{
        x.data_ptr(),
        x.grad_ptr(),
        z.grad_ptr(),
        x.len(),
        x.context(),
    });
}

// d selu(x) / d wrt is an element-wise factor times d x / d wrt; the factor is what the reverse
// kernel multiplies by, evaluated on a gradient seed of ones.
pub fn derive(args: []const OpDatum, wrt: Tensor) ?OpDatum {
    const x = args[0].tensor;
    const inner = core.derive(x, wrt) orelse return null;
    const graph = wrt.ptr;
    const factor = graph.tensor(.{ .class = .hid, .dtype = x.dtype(), .sizes = x.sizes() });
    const ones = graph.tensor(.{ .class = .hid, .dtype = x.dtype(), .sizes = x.sizes() });
    const key = core.dkey(x);
    core.invoke(core.kernels.fill, key, .{ factor.data_ptr(), 0.0, factor.len(), factor.context() });
    core.invoke(core.kernels.fill, key, .{ ones.data_ptr(), 1.0, ones.len(), ones.context() });
    core.invoke(core.kernels.selu_reverse, key, .{ x.data_ptr(), factor.data_ptr(), ones.data_ptr(), x.len(), x.context() });
    return switch (inner) {
        .scalar => |s| blk: {
            core.invoke(core.kernels.dilate, key, .{ factor.data_ptr(), s, factor.data_ptr(), factor.len(), factor.context() });
            break :blk OpDatum{ .tensor = factor };
        },
        .tensor => |t| blk: {
            core.invoke(core.kernels.hadamard, key, .{ factor.data_ptr(), t.data_ptr(), factor.data_ptr(), factor.len(), factor.context() });
            break :blk OpDatum{ .tensor = factor };
        },
        .expr => null,
    };
}
