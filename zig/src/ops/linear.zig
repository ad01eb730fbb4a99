// y = x.A + b (README.md:81,97; NOTES.md:42-45).  "ij,jk->ik" and "i,ij->j" add the bias along the output
// columns inside the contraction's epilogue; "ij,j->i" (matrix first: linear(A, x, b, ...)) has one bias entry
// per output row.  The reverse uses the native transposed-operand contractions, so no scratch transpose is
// needed (the reference transposes first, src/ops/inner_product.zig:305-330).
const std = @import("std");
const core = @import("core");
const OpDatum = core.OpDatum;
const Tensor = core.Tensor;
const Graph = core.Graph;

const Shape = struct { m: usize, n: usize, k: usize, bias_rows: bool };

fn shape_of(x: Tensor, a: Tensor, expr: []const u8) Shape {
    const xs = x.sizes();
    const as = a.sizes();
    if (std.mem.eql(u8, expr, "ij,jk->ik")) {
        std.debug.assert(xs.len == 2 and as.len == 2 and xs[1] == as[0]);
        return .{ .m = xs[0], .n = xs[1], .k = as[1], .bias_rows = false };
    } else if (std.mem.eql(u8, expr, "i,ij->j")) {
        std.debug.assert(xs.len == 1 and as.len == 2 and xs[0] == as[0]);
        return .{ .m = 1, .n = xs[0], .k = as[1], .bias_rows = false };
    } else if (std.mem.eql(u8, expr, "ij,j->i")) {
        std.debug.assert(xs.len == 2 and as.len == 1 and xs[1] == as[0]);
        return .{ .m = xs[0], .n = xs[1], .k = 1, .bias_rows = true };
    }
    @panic("Invalid expression for linear.");
}

pub fn forward(x: Tensor, a: Tensor, b: Tensor, expr: []const u8) Tensor {
    return forward_impl(x.ptr, x, a, b, expr);
}

pub fn forward_impl(graph: *Graph, x: Tensor, a: Tensor, b: Tensor, expr: []const u8) Tensor {
    const s = shape_of(x, a, expr);
    std.debug.assert(b.len() == if (s.bias_rows) s.m else s.k);

    const z = graph.tensor(.{
        .class = .hid,
        .dtype = x.dtype(),
        .sizes = if (std.mem.eql(u8, expr, "ij,jk->ik")) &.{ s.m, s.k } else if (s.bias_rows) &.{s.m} else &.{s.k},
    });
    const key = core.dkey(z);

    if (s.bias_rows) {
        core.invoke(core.kernels.inner_product_ij_jk_ik, key, .{
            x.data_ptr(), a.data_ptr(), 1.0, z.data_ptr(), 0.0, s.m, s.n, s.k, z.context(),
        });
        core.invoke(core.kernels.addition, key, .{ z.data_ptr(), b.data_ptr(), z.data_ptr(), z.len(), z.context() });
    } else {
        core.invoke(core.kernels.linear_ij_jk_ik, key, .{
            x.data_ptr(), a.data_ptr(), b.data_ptr(), 1.0, z.data_ptr(), 0.0, s.m, s.n, s.k, z.context(),
        });
    }

    if (graph.mode == .train) {
        core.attach_op(@This(), z, &.{
            OpDatum{ .tensor = x },
            OpDatum{ .tensor = a },
            OpDatum{ .tensor = b },
            OpDatum{ .expr = expr },
            OpDatum{ .tensor = z },
        });
    }
    return z;
}

// dx += G A^T ("ij,kj->ik"), dA += x^T G ("ji,jk->ik"), db += column sums of G (or G itself for "ij,j->i")
pub fn reverse(args: []const OpDatum) void {
    const x = args[0].tensor;
    const a = args[1].tensor;
    const b = args[2].tensor;
    const z = args[4].tensor;
    const s = shape_of(x, a, args[3].expr);
    const key = core.dkey(z);

    core.enable_gradient(x);
    core.enable_gradient(a);
    core.enable_gradient(b);

    core.invoke(core.kernels.inner_product_ij_kj_ik, key, .{
        z.grad_ptr(), a.data_ptr(), 1.0, x.grad_ptr(), 1.0, s.m, s.k, s.n, z.context(),
    });
    core.invoke(core.kernels.inner_product_ji_jk_ik, key, .{
        x.data_ptr(), z.grad_ptr(), 1.0, a.grad_ptr(), 1.0, s.n, s.m, s.k, z.context(),
    });
    if (s.bias_rows) {
        core.invoke(core.kernels.addition, key, .{ z.grad_ptr(), b.grad_ptr(), b.grad_ptr(), b.len(), z.context() });
    } else {
        core.invoke(core.kernels.reduce_ij_j, key, .{ z.grad_ptr(), b.grad_ptr(), 1.0, s.m, s.k, z.context() });
    }
}

// a contraction has no element-wise derivative (the reference's inner_product.derive is empty, inner_product.zig:89-90)
pub fn derive(_: []const OpDatum, _: Tensor) ?OpDatum {
    return null;
}
