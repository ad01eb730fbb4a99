// Rank-N contraction "abc,cd->abd" (NOTES.md:3-5; grammar of src/ops/expression_parsing.zig:258-317): operands of
// rank <= 6 with distinct lower-case indices in any order.  An index of both operands that is missing on the right
// is summed, one of both operands and the output is a batch index, every other index must be in the output.
// With each group flattened the contraction is C[batch][rows, columns] = A[batch][rows, summed] . B[batch][summed,
// columns]: ONE (batched) launch of the form the operands already lie in ("ij,jk" / "ij,kj" / "ji,jk"), the general
// permutation only around an operand or an output whose index order no kernel takes.  The reverse of "x,y->z" is
// the two contractions "z,y->x" and "x,z->y" through the same planner, accumulated.  Temporaries come from the
// stream's grow-only scratch (StreamEntry.get_scratch, src/core/utils.zig:20-36).
const std = @import("std");
const core = @import("core");
const OpDatum = core.OpDatum;
const Tensor = core.Tensor;
const Graph = core.Graph;

pub const MAX_RANK: usize = 6;

const Names = struct { x: []const u8, y: []const u8, z: []const u8 };

fn split(expr: []const u8) Names {
    const comma = std.mem.indexOfScalar(u8, expr, ',') orelse @panic("Invalid expression for contraction.");
    const arrow = std.mem.indexOf(u8, expr, "->") orelse @panic("Invalid expression for contraction.");
    if (comma > arrow) @panic("Invalid expression for contraction.");
    return .{ .x = expr[0..comma], .y = expr[comma + 1 .. arrow], .z = expr[arrow + 2 ..] };
}

fn has(s: []const u8, c: u8) bool {
    return std.mem.indexOfScalar(u8, s, c) != null;
}

fn check_indices(s: []const u8, rank: usize) void {
    if (s.len != rank or s.len > MAX_RANK) @panic("Contraction: the expression's rank differs from the tensor's.");
    for (s, 0..) |c, i| {
        if (c < 'a' or c > 'z') @panic("Tensor indices must be lower case characters.");
        if (std.mem.indexOfScalar(u8, s, c).? != i) @panic("Contraction: an index appears twice in one operand.");
    }
}

// a short index string built from up to three groups
const Word = struct {
    buf: [3 * MAX_RANK]u8 = undefined,
    len: usize = 0,

    fn push(self: *Word, c: u8) void {
        self.buf[self.len] = c;
        self.len += 1;
    }
    fn slice(self: *const Word) []const u8 {
        return self.buf[0..self.len];
    }
    fn join(a: []const u8, b: []const u8, c: []const u8) Word {
        var w = Word{};
        for (a) |ch| w.push(ch);
        for (b) |ch| w.push(ch);
        for (c) |ch| w.push(ch);
        return w;
    }
};

pub const Plan = struct {
    swap: bool = false, // the launch takes the operands in the opposite order; x_* then describe the caller's second operand
    kind: u2 = 0, // 0 = "ij,jk->ik", 1 = "ij,kj->ik", 2 = "ji,jk->ik" after the permutations below
    batch: usize = 0, // 0 = the rank-2 kernel
    m: usize = 1,
    n: usize = 1,
    k: usize = 1,
    x_moves: bool = false,
    y_moves: bool = false,
    z_moves: bool = false,
    x_perm: [MAX_RANK]usize = undefined, // perm[i] = new position of the operand's i-th index
    y_perm: [MAX_RANK]usize = undefined,
    z_perm: [MAX_RANK]usize = undefined, // from the launch's [batch.., rows.., columns..] result into the output
    z_sizes: [MAX_RANK]usize = undefined,
    z_rank: usize = 0,
    out_sizes: [MAX_RANK]usize = undefined,
    out_rank: usize = 0,
};

fn order_into(from: []const u8, to: []const u8, perm: *[MAX_RANK]usize) void {
    for (from, 0..) |c, i| perm[i] = std.mem.indexOfScalar(u8, to, c).?;
}

pub fn plan(xs: []const u8, ys: []const u8, zs: []const u8, x_sizes: []const usize, y_sizes: []const usize, may_swap: bool) Plan {
    check_indices(xs, x_sizes.len);
    check_indices(ys, y_sizes.len);
    check_indices(zs, zs.len);

    var extent = [_]usize{0} ** 26;
    for (xs, 0..) |c, i| extent[c - 'a'] = x_sizes[i];
    for (ys, 0..) |c, i| {
        if (has(xs, c) and extent[c - 'a'] != y_sizes[i]) @panic("Contraction: the operands' sizes differ at a shared index.");
        extent[c - 'a'] = y_sizes[i];
    }

    // batch, rows, columns in the output's order; summed in the first operand's order
    var b = Word{};
    var m = Word{};
    var n = Word{};
    var k = Word{};
    for (zs) |c| {
        const in_x = has(xs, c);
        const in_y = has(ys, c);
        if (in_x and in_y) b.push(c) else if (in_x) m.push(c) else if (in_y) n.push(c) else @panic("Contraction: an output index is in neither operand.");
    }
    for (xs) |c| {
        if (!has(zs, c)) {
            if (!has(ys, c)) @panic("Contraction: an index of one operand only must be in the output.");
            k.push(c);
        }
    }
    for (ys) |c| {
        if (!has(zs, c) and !has(xs, c)) @panic("Contraction: an index of one operand only must be in the output.");
    }

    const z_lies = Word.join(b.slice(), m.slice(), n.slice());
    const z_turned = Word.join(b.slice(), n.slice(), m.slice());
    // the output lists the second operand's indices first: C^T = B^T A^T, the same contraction with the operands exchanged
    if (may_swap and m.len != 0 and n.len != 0 and !std.mem.eql(u8, zs, z_lies.slice()) and std.mem.eql(u8, zs, z_turned.slice())) {
        var p = plan(ys, xs, zs, y_sizes, x_sizes, false);
        p.swap = true;
        return p;
    }

    var p = Plan{};
    var batch: usize = 1;
    for (b.slice()) |c| batch *= extent[c - 'a'];
    p.batch = if (b.len == 0) 0 else batch;
    for (m.slice()) |c| p.m *= extent[c - 'a'];
    for (k.slice()) |c| p.n *= extent[c - 'a'];
    for (n.slice()) |c| p.k *= extent[c - 'a'];

    const x_rows = Word.join(b.slice(), m.slice(), k.slice());
    const x_cols = Word.join(b.slice(), k.slice(), m.slice());
    const y_rows = Word.join(b.slice(), k.slice(), n.slice());
    const y_cols = Word.join(b.slice(), n.slice(), k.slice());
    const x_a = std.mem.eql(u8, xs, x_rows.slice());
    const x_t = std.mem.eql(u8, xs, x_cols.slice());
    const y_a = std.mem.eql(u8, ys, y_rows.slice());
    const y_t = std.mem.eql(u8, ys, y_cols.slice());
    // forms the kernels take: (rows, rows) = 0, (rows, cols) = 1, (cols, rows) = 2
    if (x_a and y_a) {
        p.kind = 0;
    } else if (x_a and y_t) {
        p.kind = 1;
    } else if (x_t and y_a) {
        p.kind = 2;
    } else if (x_a or x_t) {
        p.kind = if (x_a) 0 else 2;
        p.y_moves = true;
        order_into(ys, y_rows.slice(), &p.y_perm);
    } else if (y_a or y_t) {
        p.kind = if (y_a) 0 else 1;
        p.x_moves = true;
        order_into(xs, x_rows.slice(), &p.x_perm);
    } else {
        p.kind = 0;
        p.x_moves = true;
        p.y_moves = true;
        order_into(xs, x_rows.slice(), &p.x_perm);
        order_into(ys, y_rows.slice(), &p.y_perm);
    }

    if (!std.mem.eql(u8, zs, z_lies.slice())) {
        p.z_moves = true;
        order_into(z_lies.slice(), zs, &p.z_perm);
        for (z_lies.slice(), 0..) |c, i| p.z_sizes[i] = extent[c - 'a'];
        p.z_rank = z_lies.len;
    }
    for (zs, 0..) |c, i| p.out_sizes[i] = extent[c - 'a'];
    p.out_rank = zs.len;
    if (p.out_rank == 0) { // full contraction
        p.out_sizes[0] = 1;
        p.out_rank = 1;
    }
    return p;
}

fn elem_size(key: usize) usize {
    return switch (key) {
        0 => 2,
        1 => 4,
        else => 8,
    };
}

fn volume_bytes(sizes: []const usize, elem: usize) usize {
    var v: usize = elem;
    for (sizes) |s| v *= s;
    return (v + 255) & ~@as(usize, 255);
}

fn offset_ptr(base: *anyopaque, bytes: usize) *anyopaque {
    return @ptrFromInt(@intFromPtr(base) + bytes);
}

fn gemm(key: usize, kind: u2, a: *anyopaque, b: *anyopaque, alpha: f64, c: *anyopaque, beta: f64, p: Plan, ctx: anytype) void {
    if (p.batch != 0) {
        switch (kind) {
            0 => core.invoke(core.kernels.inner_product_bij_bjk_bik, key, .{ a, b, alpha, c, beta, p.batch, p.m, p.n, p.k, ctx }),
            1 => core.invoke(core.kernels.inner_product_bij_bkj_bik, key, .{ a, b, alpha, c, beta, p.batch, p.m, p.n, p.k, ctx }),
            else => core.invoke(core.kernels.inner_product_bji_bjk_bik, key, .{ a, b, alpha, c, beta, p.batch, p.m, p.n, p.k, ctx }),
        }
        return;
    }
    switch (kind) {
        0 => core.invoke(core.kernels.inner_product_ij_jk_ik, key, .{ a, b, alpha, c, beta, p.m, p.n, p.k, ctx }),
        1 => core.invoke(core.kernels.inner_product_ij_kj_ik, key, .{ a, b, alpha, c, beta, p.m, p.n, p.k, ctx }),
        else => core.invoke(core.kernels.inner_product_ji_jk_ik, key, .{ a, b, alpha, c, beta, p.m, p.n, p.k, ctx }),
    }
}

// z[zs] = scale * sum x[xs] y[ys] + beta * z
fn run(
    graph: *Graph,
    key: usize,
    x_ptr: *anyopaque,
    x_sizes: []const usize,
    xs: []const u8,
    y_ptr: *anyopaque,
    y_sizes: []const usize,
    ys: []const u8,
    scale: f64,
    z_ptr: *anyopaque,
    zs: []const u8,
    beta: f64,
) void {
    const p = plan(xs, ys, zs, x_sizes, y_sizes, true);
    const elem = elem_size(key);
    const ctx = graph.stream.context;

    var a = if (p.swap) y_ptr else x_ptr;
    var b = if (p.swap) x_ptr else y_ptr;
    const a_sizes = if (p.swap) y_sizes else x_sizes;
    const b_sizes = if (p.swap) x_sizes else y_sizes;

    const xb = if (p.x_moves) volume_bytes(a_sizes, elem) else 0;
    const yb = if (p.y_moves) volume_bytes(b_sizes, elem) else 0;
    const zb = if (p.z_moves) volume_bytes(p.z_sizes[0..p.z_rank], elem) else 0;

    var c = z_ptr;
    if (xb + yb + zb != 0) {
        const tmp: *anyopaque = graph.stream.get_scratch(.r64, (xb + yb + zb + 7) / 8);
        if (p.x_moves) {
            core.invoke(core.kernels.permutate, key, .{ a, tmp, 0.0, a_sizes.ptr, &p.x_perm, a_sizes.len, ctx });
            a = tmp;
        }
        if (p.y_moves) {
            const moved = offset_ptr(tmp, xb);
            core.invoke(core.kernels.permutate, key, .{ b, moved, 0.0, b_sizes.ptr, &p.y_perm, b_sizes.len, ctx });
            b = moved;
        }
        if (p.z_moves) c = offset_ptr(tmp, xb + yb);
    }

    gemm(key, p.kind, a, b, scale, c, if (p.z_moves) 0.0 else beta, p, ctx);

    if (p.z_moves) {
        core.invoke(core.kernels.permutate, key, .{ c, z_ptr, beta, &p.z_sizes, &p.z_perm, p.z_rank, ctx });
    }
}

pub fn forward(x: Tensor, y: Tensor, expr: []const u8) Tensor {
    return forward_scaled(x, y, 1.0, expr);
}

pub fn forward_scaled(x: Tensor, y: Tensor, scale: f64, expr: []const u8) Tensor {
    return forward_impl(x.ptr, x, y, scale, expr);
}

pub fn forward_impl(graph: *Graph, x: Tensor, y: Tensor, scale: f64, expr: []const u8) Tensor {
    std.debug.assert(x.dtype() == y.dtype());
    const e = split(expr);
    const p = plan(e.x, e.y, e.z, x.sizes(), y.sizes(), true);

    const z = graph.tensor(.{ .class = .hid, .dtype = x.dtype(), .sizes = p.out_sizes[0..p.out_rank] });

    run(graph, core.dkey(z), x.data_ptr(), x.sizes(), e.x, y.data_ptr(), y.sizes(), e.y, scale, z.data_ptr(), e.z, 0.0);

    if (graph.mode == .train) {
        core.attach_op(@This(), z, &.{
            OpDatum{ .tensor = x },
            OpDatum{ .tensor = y },
            OpDatum{ .scalar = scale },
            OpDatum{ .expr = expr },
            OpDatum{ .tensor = z },
        });
    }
    return z;
}

// dX += scale * (dZ contracted with Y over the indices X lacks), dY += scale * (X contracted with dZ)
pub fn reverse(args: []const OpDatum) void {
    const x = args[0].tensor;
    const y = args[1].tensor;
    const scale = args[2].scalar;
    const e = split(args[3].expr);
    const z = args[4].tensor;
    const key = core.dkey(z);

    core.enable_gradient(x);
    core.enable_gradient(y);

    // a full contraction is stored as one element; its index string is empty
    const z_sizes: []const usize = if (e.z.len == 0) &.{} else z.sizes();

    run(z.ptr, key, z.grad_ptr(), z_sizes, e.z, y.data_ptr(), y.sizes(), e.y, scale, x.grad_ptr(), e.x, 1.0);
    run(z.ptr, key, x.data_ptr(), x.sizes(), e.x, z.grad_ptr(), z_sizes, e.z, scale, y.grad_ptr(), e.y, 1.0);
}

// a contraction has no element-wise derivative (the reference's inner_product.derive is empty, inner_product.zig:89-90)
pub fn derive(_: []const OpDatum, _: Tensor) ?OpDatum {
    return null;
}
