// Mamba-2 SSD scan: y_t = C_t^T S_t with S_t = exp(dt_t A_h) S_{t-1} + dt_t B_t x_t^T per (batch, head).
// x: [batch, seqlen, heads, headdim], dt: [batch, seqlen, heads] (after softplus), A: [heads] (negative),
// B, C: [batch, seqlen, groups, dstate].  r16 storage runs on the tensor-core kernels, r32 / r64 on the
// sequential-recurrence kernels behind the same launcher names.
const std = @import("std");
const core = @import("core");
const OpDatum = core.OpDatum;
const Tensor = core.Tensor;
const Graph = core.Graph;
const C = @import("../core/cimport.zig").C;

const Dims = struct { batch: usize, seqlen: usize, heads: usize, headdim: usize, dstate: usize, groups: usize };

fn scratch_bytes(key: usize, d: Dims, chunk: usize, reverse_pass: u32) usize {
    if (key == 0) return C.mpSsdScanScratchBytes(d.batch, d.seqlen, d.heads, d.headdim, d.dstate, d.groups, chunk, reverse_pass);
    return C.mpSsdScanGenericScratchBytes(@intCast(key), d.batch, d.seqlen, d.heads, d.headdim, d.dstate, d.groups, reverse_pass);
}

fn dims_of(x: Tensor, b: Tensor) Dims {
    const xs = x.sizes();
    const bs = b.sizes();
    std.debug.assert(xs.len == 4 and bs.len == 4 and bs[0] == xs[0] and bs[1] == xs[1]);
    return .{ .batch = xs[0], .seqlen = xs[1], .heads = xs[2], .headdim = xs[3], .dstate = bs[3], .groups = bs[2] };
}

pub fn forward(x: Tensor, dt: Tensor, a: Tensor, b: Tensor, c: Tensor, chunk: usize) Tensor {
    return forward_impl(x.ptr, x, dt, a, b, c, chunk);
}

pub fn forward_impl(graph: *Graph, x: Tensor, dt: Tensor, a: Tensor, b: Tensor, c: Tensor, chunk: usize) Tensor {
    const d = dims_of(x, b);
    const y = graph.tensor(.{ .class = .hid, .dtype = x.dtype(), .sizes = x.sizes() });
    const key = core.dkey(y);

    const scratch = graph.stream.get_scratch(.r64, (scratch_bytes(key, d, chunk, 0) + 7) / 8);

    core.invoke(core.kernels.ssd_scan, key, .{
        x.data_ptr(), dt.data_ptr(), a.data_ptr(), b.data_ptr(), c.data_ptr(), y.data_ptr(), scratch,
        d.batch, d.seqlen, d.heads, d.headdim, d.dstate, d.groups, chunk, y.context(),
    });

    if (graph.mode == .train) {
        core.attach_op(@This(), y, &.{
            OpDatum{ .tensor = x },
            OpDatum{ .tensor = dt },
            OpDatum{ .tensor = a },
            OpDatum{ .tensor = b },
            OpDatum{ .tensor = c },
            OpDatum{ .scalar = @floatFromInt(chunk) },
            OpDatum{ .tensor = y },
        });
    }
    return y;
}

// The launcher overwrites its outputs, so the gradients of this op go to temporaries of the graph's allocator
// and are then added to the accumulated gradients (g = g_new + g), like every other reverse of the reference.
pub fn reverse(args: []const OpDatum) void {
    const x = args[0].tensor;
    const dt = args[1].tensor;
    const a = args[2].tensor;
    const b = args[3].tensor;
    const c = args[4].tensor;
    const chunk: usize = @intFromFloat(args[5].scalar);
    const y = args[6].tensor;
    const graph = y.ptr;
    const d = dims_of(x, b);

    inline for (.{ x, dt, a, b, c }) |t| core.enable_gradient(t);

    const gx = graph.tensor(.{ .class = .hid, .dtype = x.dtype(), .sizes = x.sizes() });
    const gdt = graph.tensor(.{ .class = .hid, .dtype = dt.dtype(), .sizes = dt.sizes() });
    const ga = graph.tensor(.{ .class = .hid, .dtype = a.dtype(), .sizes = a.sizes() });
    const gb = graph.tensor(.{ .class = .hid, .dtype = b.dtype(), .sizes = b.sizes() });
    const gc = graph.tensor(.{ .class = .hid, .dtype = c.dtype(), .sizes = c.sizes() });

    const key = core.dkey(y);
    const scratch = graph.stream.get_scratch(.r64, (scratch_bytes(key, d, chunk, 1) + 7) / 8);

    core.invoke(core.kernels.ssd_scan_reverse, key, .{
        x.data_ptr(), dt.data_ptr(), a.data_ptr(), b.data_ptr(), c.data_ptr(), y.grad_ptr(),
        gx.data_ptr(), gdt.data_ptr(), ga.data_ptr(), gb.data_ptr(), gc.data_ptr(), scratch,
        d.batch, d.seqlen, d.heads, d.headdim, d.dstate, d.groups, chunk, y.context(),
    });

    inline for (.{ .{ gx, x }, .{ gdt, dt }, .{ ga, a }, .{ gb, b }, .{ gc, c } }) |pair| {
        core.invoke(core.kernels.addition, core.dkey(pair[1]), .{
            pair[0].data_ptr(),
            pair[1].grad_ptr(),
            pair[1].grad_ptr(),
            pair[1].len(),
            pair[1].context(),
        });
        pair[0].free();
    }
}

pub fn derive(_: []const OpDatum, _: Tensor) ?OpDatum {
    return null;
}
