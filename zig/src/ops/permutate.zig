// Any permutation of a tensor of rank <= 6 ("ij->ji", "ijk->kij", ... NOTES.md:3-5; grammar of
// src/ops/expression_parsing.zig:205-255).  Replaces src/ops/permutate.zig, whose map holds "ij->ji" only.
// dst[perm(i)] = src[i] + alpha * dst[perm(i)]; with alpha = 0 the destination is not read and the result is
// bit-exact.  The reverse applies the inverse permutation to the upstream gradient with alpha = 1.
const std = @import("std");
const core = @import("core");
const OpDatum = core.OpDatum;
const Tensor = core.Tensor;
const Graph = core.Graph;

pub const MAX_RANK: usize = 6;

pub const Permutation = struct {
    rank: usize,
    perm: [MAX_RANK]usize, // perm[i] = position of the i-th input index in the output

    pub fn parse(expr: []const u8) Permutation {
        const arrow = std.mem.indexOf(u8, expr, "->") orelse @panic("Invalid expression for permutate.");
        const lhs = expr[0..arrow];
        const rhs = expr[arrow + 2 ..];
        if (lhs.len != rhs.len or lhs.len == 0 or lhs.len > MAX_RANK) @panic("Invalid expression for permutate.");
        var p = Permutation{ .rank = lhs.len, .perm = undefined };
        for (lhs, 0..) |ch, i| {
            p.perm[i] = std.mem.indexOfScalar(u8, rhs, ch) orelse @panic("Index missing on the right of permutate expression.");
        }
        return p;
    }

    pub fn inverse(self: Permutation) Permutation {
        var q = Permutation{ .rank = self.rank, .perm = undefined };
        for (0..self.rank) |i| q.perm[self.perm[i]] = i;
        return q;
    }
};

pub fn forward(x: Tensor, expr: []const u8) Tensor {
    return forward_impl(x.ptr, x, expr);
}

pub fn forward_impl(graph: *Graph, x: Tensor, expr: []const u8) Tensor {
    const p = Permutation.parse(expr);
    const xs = x.sizes();
    std.debug.assert(xs.len == p.rank);

    var ys: [MAX_RANK]usize = undefined;
    for (0..p.rank) |i| ys[p.perm[i]] = xs[i];

    const y = graph.tensor(.{ .class = .hid, .dtype = x.dtype(), .sizes = ys[0..p.rank] });

    core.invoke(core.kernels.permutate, core.dkey(x), .{
        x.data_ptr(),
        y.data_ptr(),
        0.0,
        xs.ptr,
        &p.perm,
        p.rank,
        graph.stream.context,
    });

    if (graph.mode == .train) {
        core.attach_op(@This(), y, &.{
            OpDatum{ .tensor = x },
            OpDatum{ .tensor = y },
            OpDatum{ .expr = expr },
        });
    }
    return y;
}

pub fn reverse(args: []const OpDatum) void {
    const x = args[0].tensor;
    const y = args[1].tensor;
    const q = Permutation.parse(args[2].expr).inverse();

    core.enable_gradient(x);

    core.invoke(core.kernels.permutate, core.dkey(x), .{
        y.grad_ptr(),
        x.grad_ptr(),
        1.0,
        y.sizes().ptr,
        &q.perm,
        q.rank,
        y.ptr.stream.context,
    });
}

// the derivative of a permuted tensor is the permuted derivative (the reference panics here, permutate.zig:71-73)
pub fn derive(args: []const OpDatum, wrt: Tensor) ?OpDatum {
    const inner = core.derive(args[0].tensor, wrt) orelse return null;
    return switch (inner) {
        .scalar => inner,
        .tensor => |t| OpDatum{ .tensor = forward_impl(wrt.ptr, t, args[2].expr) },
        .expr => null,
    };
}
