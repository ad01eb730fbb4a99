//! Scalar Zig host oracle of the op-kernel layer: one plain loop per op, sums in f64.
//!
//! TEST INFRASTRUCTURE, kept as source: no Zig toolchain exists where this repository is built, so the
//! executable oracle is the C twin beside it (oracle/oracle.c, oracle/oracle_body.inc: same loops, same
//! accumulation choices) and this file is what a Metaphor checkout compiles (`zig test oracle/zig/oracle.zig`).
//! Each function names the reference kernel body it restates, or says that the reference has none.
const std = @import("std");

fn Acc(comptime T: type) type {
    return if (T == f64) f64 else f32; // r16 / r32 compute in f32, r64 in f64 (the library's kernels do the same)
}

// ---- flat element-wise (src/cuda/nvcc_src/{addition,subtraction,hadamard,hadamard_reverse}.cu:12) ----------
pub fn addition(comptime T: type, a: []const T, b: []const T, c: []T) void {
    for (a, b, c) |x, y, *z| z.* = x + y;
}
pub fn subtraction(comptime T: type, a: []const T, b: []const T, c: []T) void {
    for (a, b, c) |x, y, *z| z.* = x - y;
}
pub fn hadamard(comptime T: type, a: []const T, b: []const T, c: []T) void {
    for (a, b, c) |x, y, *z| z.* = x * y;
}
pub fn hadamard_reverse(comptime T: type, a: []const T, b: []const T, c: []T) void {
    for (a, b, c) |x, y, *z| z.* += x * y;
}
// negate.cu:11, translate.cu:12, dilate.cu:12, dilate_reverse.cu:12
pub fn negate(comptime T: type, a: []const T, b: []T) void {
    for (a, b) |x, *y| y.* = -x;
}
pub fn translate(comptime T: type, a: []const T, value: f64, b: []T) void {
    const v: T = @floatCast(value);
    for (a, b) |x, *y| y.* = x + v;
}
pub fn dilate(comptime T: type, a: []const T, value: f64, b: []T) void {
    const v: T = @floatCast(value);
    for (a, b) |x, *y| y.* = x * v;
}
pub fn dilate_reverse(comptime T: type, a: []const T, value: f64, b: []T) void {
    const v: T = @floatCast(value);
    for (a, b) |x, *y| y.* += x * v;
}
// relu.cu:11-12, relu_reverse.cu:12-14; stepwise is a true step here (the reference body copies relu, stepwise.cu:11-12)
pub fn relu(comptime T: type, a: []const T, b: []T) void {
    for (a, b) |x, *y| y.* = if (x >= 0) x else 0;
}
pub fn relu_reverse(comptime T: type, a: []const T, ga: []T, gb: []const T) void {
    for (a, ga, gb) |x, *g, u| {
        if (x >= 0) g.* += u;
    }
}
pub fn stepwise(comptime T: type, a: []const T, b: []T) void {
    for (a, b) |x, *y| y.* = if (x >= 0) 1 else 0;
}
// fill.cu:12, sequence.cu:14 (evaluated in T), copy.cu:20-29
pub fn fill(comptime T: type, a: []T, value: f64) void {
    const v: T = @floatCast(value);
    for (a) |*x| x.* = v;
}
pub fn sequence(comptime T: type, a: []T, init: f64, step: f64) void {
    const i0: T = @floatCast(init);
    const st: T = @floatCast(step);
    for (a, 0..) |*x, i| x.* = i0 + st * @as(T, @floatFromInt(i));
}
pub fn copy(comptime T: type, src: []const T, dst: []T) void {
    @memcpy(dst, src);
}

// ---- selu (no reference kernel; README.md:97) ---------------------------------------------------------------
pub const selu_lambda: f64 = 1.0507009873554805;
pub const selu_alpha: f64 = 1.6732632423543772;
pub fn selu(comptime T: type, a: []const T, b: []T) void {
    for (a, b) |x, *y| {
        const v: f64 = x;
        y.* = @floatCast(selu_lambda * (if (v > 0) v else selu_alpha * (@exp(v) - 1.0)));
    }
}
pub fn selu_reverse(comptime T: type, a: []const T, ga: []T, gb: []const T) void {
    for (a, ga, gb) |x, *g, u| {
        const v: f64 = x;
        const d = selu_lambda * (if (v > 0) 1.0 else selu_alpha * @exp(v));
        g.* += @floatCast(@as(f64, u) * d);
    }
}

// ---- rank 2 (permutate_ij_ji.cu:22-40, reduce_ij_i.cu:20-32, reduce_ij_j.cu:19-44 as a formula, broadcast_*.cu) ----
pub fn permutate_ij_ji(comptime T: type, src: []const T, dst: []T, alpha: f64, m: usize, n: usize) void {
    for (0..m) |i| for (0..n) |j| {
        const old: f64 = if (alpha != 0) @as(f64, dst[j * m + i]) * alpha else 0; // alpha = 0 never reads dst
        dst[j * m + i] = @floatCast(@as(f64, src[i * n + j]) + old);
    };
}
pub fn reduce_ij_i(comptime T: type, src: []const T, dst: []T, alpha: f64, m: usize, n: usize) void {
    for (0..m) |i| {
        var s: f64 = 0;
        for (0..n) |j| s += src[i * n + j];
        dst[i] = @floatCast(s + (if (alpha != 0) alpha * @as(f64, dst[i]) else 0));
    }
}
pub fn reduce_ij_j(comptime T: type, src: []const T, dst: []T, alpha: f64, m: usize, n: usize) void {
    for (0..n) |j| {
        var s: f64 = 0;
        for (0..m) |i| s += src[i * n + j];
        dst[j] = @floatCast(s + (if (alpha != 0) alpha * @as(f64, dst[j]) else 0));
    }
}
pub fn broadcast_i_ij(comptime T: type, src: []const T, dst: []T, alpha: f64, m: usize, n: usize) void {
    for (0..m) |i| for (0..n) |j| {
        dst[i * n + j] = @floatCast(@as(f64, src[i]) + (if (alpha != 0) alpha * @as(f64, dst[i * n + j]) else 0));
    };
}
pub fn broadcast_j_ij(comptime T: type, src: []const T, dst: []T, alpha: f64, m: usize, n: usize) void {
    for (0..m) |i| for (0..n) |j| {
        dst[i * n + j] = @floatCast(@as(f64, src[j]) + (if (alpha != 0) alpha * @as(f64, dst[i * n + j]) else 0));
    };
}

// ---- contractions: C[m,k] = alpha op(A)[m,n] op(B)[n,k] + bias[k] + beta C (inner_product_ij_jk_ik.cu:12-26;
//      the arithmetic itself lives in cuBLAS in the reference) -------------------------------------------------------
pub fn inner_product(comptime T: type, a: []const T, b: []const T, bias: ?[]const T, alpha: f64, c: []T, beta: f64,
                     m: usize, n: usize, k: usize, ta: bool, tb: bool) void {
    for (0..m) |i| for (0..k) |l| {
        var s: f64 = 0;
        for (0..n) |j| {
            const x: f64 = if (ta) a[j * m + i] else a[i * n + j];
            const y: f64 = if (tb) b[l * n + j] else b[j * k + l];
            s += x * y;
        }
        var r = alpha * s;
        if (bias) |bv| r += bv[l];
        if (beta != 0) r += beta * @as(f64, c[i * k + l]);
        c[i * k + l] = @floatCast(r);
    };
}

// ---- row-wise softmax and RMSNorm (no reference kernels) ------------------------------------------------------------
pub fn softmax_ij_j(comptime T: type, x: []const T, y: []T, m: usize, n: usize) void {
    for (0..m) |i| {
        var mx: f64 = -std.math.inf(f64);
        for (0..n) |j| mx = @max(mx, @as(f64, x[i * n + j]));
        var s: f64 = 0;
        for (0..n) |j| s += @exp(@as(f64, x[i * n + j]) - mx);
        for (0..n) |j| y[i * n + j] = @floatCast(@exp(@as(f64, x[i * n + j]) - mx) / s);
    }
}
// gx = y o (gy - sum_j gy o y) + alpha gx
pub fn softmax_ij_j_reverse(comptime T: type, y: []const T, gy: []const T, gx: []T, alpha: f64, m: usize, n: usize) void {
    for (0..m) |i| {
        var d: f64 = 0;
        for (0..n) |j| d += @as(f64, gy[i * n + j]) * @as(f64, y[i * n + j]);
        for (0..n) |j| {
            const r = @as(f64, y[i * n + j]) * (@as(f64, gy[i * n + j]) - d);
            gx[i * n + j] = @floatCast(r + (if (alpha != 0) alpha * @as(f64, gx[i * n + j]) else 0));
        }
    }
}
pub fn rmsnorm_ij_j(comptime T: type, x: []const T, gain: []const T, eps: f64, y: []T, rstd: ?[]Acc(T), m: usize, n: usize) void {
    for (0..m) |i| {
        var ss: f64 = 0;
        for (0..n) |j| ss += @as(f64, x[i * n + j]) * @as(f64, x[i * n + j]);
        const r = 1.0 / @sqrt(ss / @as(f64, @floatFromInt(n)) + eps);
        if (rstd) |rs| rs[i] = @floatCast(r);
        for (0..n) |j| y[i * n + j] = @floatCast(@as(f64, x[i * n + j]) * r * @as(f64, gain[j]));
    }
}
// gx = r (gy o gain) - x r^3 mean_j(gy o gain o x) + alpha gx;  ggain = sum_i gy o x r_i + alpha ggain
pub fn rmsnorm_ij_j_reverse(comptime T: type, x: []const T, gain: []const T, gy: []const T, eps: f64, gx: []T, ggain: []T,
                            alpha: f64, m: usize, n: usize, col_sums: []f64) void {
    @memset(col_sums, 0);
    const inv_n = 1.0 / @as(f64, @floatFromInt(n));
    for (0..m) |i| {
        var ss: f64 = 0;
        var dot: f64 = 0;
        for (0..n) |j| {
            const xv: f64 = x[i * n + j];
            ss += xv * xv;
            dot += @as(f64, gy[i * n + j]) * @as(f64, gain[j]) * xv;
        }
        const r = 1.0 / @sqrt(ss * inv_n + eps);
        for (0..n) |j| {
            const xv: f64 = x[i * n + j];
            const g: f64 = gy[i * n + j];
            const v = r * g * @as(f64, gain[j]) - xv * r * r * r * dot * inv_n;
            gx[i * n + j] = @floatCast(v + (if (alpha != 0) alpha * @as(f64, gx[i * n + j]) else 0));
            col_sums[j] += g * xv * r;
        }
    }
    for (0..n) |j| ggain[j] = @floatCast(col_sums[j] + (if (alpha != 0) alpha * @as(f64, ggain[j]) else 0));
}

// ---- optimizer steps (intent of src/optm/optimizer.zig:160-179; Adam: NOTES.md:11) --------------------------------------
pub fn sgd(comptime T: type, w: []T, g: []const T, rate: f64, lo: f64, hi: f64) void {
    for (w, g) |*wv, gv| wv.* = @floatCast(@as(f64, wv.*) - rate * @min(@max(@as(f64, gv), lo), hi));
}
pub fn adam(comptime T: type, w: []T, g: []const T, m: []T, v: []T, lr: f64, b1: f64, b2: f64, eps: f64, grad_scale: f64, step: usize) void {
    const t: f64 = @floatFromInt(@max(step, 1));
    const c1 = 1.0 - std.math.pow(f64, b1, t);
    const c2 = 1.0 - std.math.pow(f64, b2, t);
    for (w, g, m, v) |*wv, gv, *mv, *vv| {
        const gs = @as(f64, gv) * grad_scale;
        const mn = b1 * @as(f64, mv.*) + (1.0 - b1) * gs;
        const vn = b2 * @as(f64, vv.*) + (1.0 - b2) * gs * gs;
        wv.* = @floatCast(@as(f64, wv.*) - lr * (mn / c1) / (@sqrt(vn / c2) + eps));
        mv.* = @floatCast(mn);
        vv.* = @floatCast(vn);
    }
}

// ---- Mamba-2 SSD scan, sequential recurrence in f64 (no reference kernel) ---------------------------------------------
// x, y: [batch, L, H, P]; dt: [batch, L, H]; A: [H]; B, C: [batch, L, G, N].  S_t = exp(dt_t A_h) S_{t-1} + dt_t B_t x_t^T,
// y_t = C_t^T S_t.  `state` is caller scratch of N*P values.
pub fn ssd_forward(x: []const f64, dt: []const f64, a: []const f64, bm: []const f64, cm: []const f64, y: []f64,
                   batch: usize, len: usize, heads: usize, p: usize, n: usize, groups: usize, state: []f64) void {
    const hpg = heads / groups;
    for (0..batch) |b| for (0..heads) |h| {
        @memset(state, 0);
        const g = h / hpg;
        for (0..len) |t| {
            const d = dt[(b * len + t) * heads + h];
            const decay = @exp(d * a[h]);
            const xb = ((b * len + t) * heads + h) * p;
            const gb = ((b * len + t) * groups + g) * n;
            for (0..n) |i| for (0..p) |j| {
                state[i * p + j] = decay * state[i * p + j] + d * bm[gb + i] * x[xb + j];
            };
            for (0..p) |j| {
                var s: f64 = 0;
                for (0..n) |i| s += cm[gb + i] * state[i * p + j];
                y[xb + j] = s;
            }
        }
    };
}

// Adjoint recurrence, t = L-1 .. 0 with lambda_t = C_t gy_t^T + exp(dt_{t+1} A) lambda_{t+1}:
//   gC_t += S_t gy_t, gx_t = dt_t lambda_t^T B_t, gB_t += dt_t lambda_t x_t,
//   gdt_t = <lambda_t, B_t x_t^T> + A exp(dt_t A) <lambda_t, S_{t-1}>, gA += dt_t exp(dt_t A) <lambda_t, S_{t-1}>.
// `states` is caller scratch of (L+1)*N*P values (the forward states of one sequence), `lambda` of N*P.
pub fn ssd_reverse(x: []const f64, dt: []const f64, a: []const f64, bm: []const f64, cm: []const f64, gy: []const f64,
                   gx: []f64, gdt: []f64, ga: []f64, gb_out: []f64, gc_out: []f64,
                   batch: usize, len: usize, heads: usize, p: usize, n: usize, groups: usize, states: []f64, lambda: []f64) void {
    const hpg = heads / groups;
    const np = n * p;
    @memset(ga, 0);
    @memset(gb_out, 0);
    @memset(gc_out, 0);
    for (0..batch) |b| for (0..heads) |h| {
        const g = h / hpg;
        @memset(states[0..np], 0);
        for (0..len) |t| {
            const d = dt[(b * len + t) * heads + h];
            const decay = @exp(d * a[h]);
            const xb = ((b * len + t) * heads + h) * p;
            const gbase = ((b * len + t) * groups + g) * n;
            for (0..n) |i| for (0..p) |j| {
                states[(t + 1) * np + i * p + j] = decay * states[t * np + i * p + j] + d * bm[gbase + i] * x[xb + j];
            };
        }
        @memset(lambda, 0);
        var t: usize = len;
        while (t > 0) {
            t -= 1;
            const d = dt[(b * len + t) * heads + h];
            const decay = @exp(d * a[h]);
            const xb = ((b * len + t) * heads + h) * p;
            const gbase = ((b * len + t) * groups + g) * n;
            if (t + 1 < len) {
                const dn = @exp(dt[(b * len + t + 1) * heads + h] * a[h]);
                for (lambda) |*l| l.* *= dn;
            }
            for (0..n) |i| for (0..p) |j| {
                lambda[i * p + j] += cm[gbase + i] * gy[xb + j];
            };
            var direct: f64 = 0;
            var carried: f64 = 0;
            for (0..n) |i| {
                var sc: f64 = 0;
                var sb: f64 = 0;
                for (0..p) |j| {
                    sc += states[(t + 1) * np + i * p + j] * gy[xb + j];
                    sb += lambda[i * p + j] * x[xb + j];
                    carried += lambda[i * p + j] * states[t * np + i * p + j];
                }
                gc_out[gbase + i] += sc;
                gb_out[gbase + i] += d * sb;
                direct += bm[gbase + i] * sb;
            }
            for (0..p) |j| {
                var s: f64 = 0;
                for (0..n) |i| s += lambda[i * p + j] * bm[gbase + i];
                gx[xb + j] = d * s;
            }
            gdt[(b * len + t) * heads + h] = direct + a[h] * decay * carried;
            ga[h] += d * decay * carried;
        }
    };
}

// ---- pins: hand-derivable values of src/examples/experimental.zig:19-69 ------------------------------------------------
test "hadamard of sums and its reverse" {
    // e = (a + b) * (c + d) with a = 1, b = 2, c = 3, d = 4: e = 21; de/da = de/db = 7, de/dc = de/dd = 3
    var a = [_]f32{1}; var b = [_]f32{2}; var c = [_]f32{3}; var d = [_]f32{4};
    var s1: [1]f32 = undefined; var s2: [1]f32 = undefined; var e: [1]f32 = undefined;
    addition(f32, &a, &b, &s1);
    addition(f32, &c, &d, &s2);
    hadamard(f32, &s1, &s2, &e);
    try std.testing.expectEqual(@as(f32, 21), e[0]);
    var g1 = [_]f32{0}; var g2 = [_]f32{0}; const seed = [_]f32{1};
    hadamard_reverse(f32, &seed, &s2, &g1);
    hadamard_reverse(f32, &seed, &s1, &g2);
    try std.testing.expectEqual(@as(f32, 7), g1[0]);
    try std.testing.expectEqual(@as(f32, 3), g2[0]);
}

test "softmax rows sum to one and its reverse is orthogonal to ones" {
    const x = [_]f64{ 0.5, -1.0, 2.0, 0.0, 0.0, 0.0 };
    var y: [6]f64 = undefined;
    softmax_ij_j(f64, &x, &y, 2, 3);
    try std.testing.expectApproxEqAbs(@as(f64, 1), y[0] + y[1] + y[2], 1e-12);
    try std.testing.expectApproxEqAbs(@as(f64, 1.0 / 3.0), y[4], 1e-12);
    const gy = [_]f64{ 1, 2, 3, 4, 5, 6 };
    var gx: [6]f64 = undefined;
    softmax_ij_j_reverse(f64, &y, &gy, &gx, 0, 2, 3);
    try std.testing.expectApproxEqAbs(@as(f64, 0), gx[0] + gx[1] + gx[2], 1e-12);
}
