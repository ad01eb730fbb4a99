// The gated norm of a Mamba-2 block in one launch each way:
//   u = (y + D[h] x) * silu(z),   out = u * rsqrt(mean_j u^2 + eps) * gain
// y, x: [rows, heads * headdim] (the scan's output and input); z: the gate, a column slice of a wider matrix
// (pointer + row pitch in elements); D: per-head skip factors in the accumulator type; gain: [heads * headdim].
// The gated activation u is never stored: the reverse recomputes it from y, x and z, so only rstd (one value per
// row, accumulator type) is kept between the passes.
const std = @import("std");
const core = @import("core");
const OpDatum = core.OpDatum;
const Tensor = core.Tensor;
const Graph = core.Graph;
const C = @import("../core/cimport.zig").C;

pub fn forward(y: Tensor, x: Tensor, d: Tensor, z: Tensor, z_pitch: usize, gain: Tensor, eps: f64, heads: usize) Tensor {
    return forward_impl(y.ptr, y, x, d, z, z_pitch, gain, eps, heads);
}

pub fn forward_impl(graph: *Graph, y: Tensor, x: Tensor, d: Tensor, z: Tensor, z_pitch: usize, gain: Tensor, eps: f64, heads: usize) Tensor {
    const ys = y.sizes();
    std.debug.assert(ys.len == 2 and ys[1] % heads == 0 and gain.len() == ys[1] and d.len() == heads);
    const headdim = ys[1] / heads;

    const out = graph.tensor(.{ .class = .hid, .dtype = y.dtype(), .sizes = ys });
    const rstd = graph.tensor(.{ .class = .hid, .dtype = d.dtype(), .sizes = &.{ys[0]} });

    core.invoke(core.kernels.ssd_gate_rmsnorm, core.dkey(out), .{
        y.data_ptr(), x.data_ptr(), d.data_ptr(), z.data_ptr(), z_pitch, gain.data_ptr(), eps,
        out.data_ptr(), rstd.data_ptr(), ys[0], heads, headdim, out.context(),
    });

    if (graph.mode == .train) {
        core.attach_op(@This(), out, &.{
            OpDatum{ .tensor = y },
            OpDatum{ .tensor = x },
            OpDatum{ .tensor = d },
            OpDatum{ .tensor = z },
            OpDatum{ .scalar = @floatFromInt(z_pitch) },
            OpDatum{ .tensor = gain },
            OpDatum{ .tensor = rstd },
            OpDatum{ .scalar = @floatFromInt(heads) },
            OpDatum{ .tensor = out },
        });
    }
    return out;
}

// The launcher overwrites g_y and g_z and accumulates g_D; g_gain is blended with alpha = 1.  g_y and g_z go to
// temporaries that are then added to the accumulated gradients, like every other reverse of the reference; the skip's
// share of g_x (D[h] * g_y) is added by head_scale_accumulate.
pub fn reverse(args: []const OpDatum) void {
    const y = args[0].tensor;
    const x = args[1].tensor;
    const d = args[2].tensor;
    const z = args[3].tensor;
    const z_pitch: usize = @intFromFloat(args[4].scalar);
    const gain = args[5].tensor;
    const rstd = args[6].tensor;
    const heads: usize = @intFromFloat(args[7].scalar);
    const out = args[8].tensor;
    const graph = out.ptr;
    const ys = y.sizes();
    const headdim = ys[1] / heads;

    inline for (.{ y, x, d, z, gain }) |t| core.enable_gradient(t);

    const gy = graph.tensor(.{ .class = .hid, .dtype = y.dtype(), .sizes = ys });
    const gz = graph.tensor(.{ .class = .hid, .dtype = y.dtype(), .sizes = ys });

    const bytes = C.mpSsdGateRmsnormReverseScratchBytes(ys[0], heads, headdim, out.context());
    const scratch = graph.stream.get_scratch(.r64, (bytes + 7) / 8);

    core.invoke(core.kernels.ssd_gate_rmsnorm_reverse, core.dkey(out), .{
        y.data_ptr(), x.data_ptr(), d.data_ptr(), z.data_ptr(), z_pitch, gain.data_ptr(), rstd.data_ptr(), out.grad_ptr(),
        gy.data_ptr(), gz.data_ptr(), ys[1], d.grad_ptr(), gain.grad_ptr(), 1.0, scratch, ys[0], heads, headdim, out.context(),
    });

    // g_x += D[h] * g_y, then g_y joins y's gradient
    core.invoke(core.kernels.head_scale_accumulate, core.dkey(out), .{
        d.data_ptr(), gy.data_ptr(), x.grad_ptr(), ys[0], heads, headdim, out.context(),
    });
    core.invoke(core.kernels.addition, core.dkey(y), .{ gy.data_ptr(), y.grad_ptr(), y.grad_ptr(), y.len(), y.context() });
    gy.free();

    // This wrapper accumulates z's gradient only for a dense z (z_pitch == width).  A host that keeps z as a column slice
    // of the projection's output passes the slice of that output's gradient as gz with the same pitch and lets the
    // launcher write it in place (what metaphor_b200/mamba_lm.py does).
    std.debug.assert(z_pitch == ys[1]);
    core.invoke(core.kernels.addition, core.dkey(z), .{ gz.data_ptr(), z.grad_ptr(), z.grad_ptr(), z.len(), z.context() });
    gz.free();
}

pub fn derive(_: []const OpDatum, _: Tensor) ?OpDatum {
    return null;
}
