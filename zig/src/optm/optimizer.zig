// Optimizers over the library's fused update kernels.  Refresh of src/optm/optimizer.zig: its SGD (:126-180)
// and Momentum (:182-275) call `overloads.kernel_gradient_descent` / `kernel_momentum`, which do not exist in
// the reference's device layer; Adam is only named in NOTES.md:11.  One launch per weight tensor, one stream
// synchronisation at the end (the reference synchronises every stream it touched, :151-154).
const std = @import("std");
const core = @import("core");
const Graph = core.Graph;
const Tensor = core.Tensor;

pub const ClipRange = struct {
    lower: f64,
    upper: f64,

    pub fn init() ClipRange {
        return .{ .lower = -std.math.inf(f64), .upper = std.math.inf(f64) };
    }
};

// walks the leaf block and hands every weight that has a gradient to `f`
fn for_each_weight(graph: *Graph, ctx: anytype, comptime f: anytype) void {
    const block = &graph.leaf_block;
    for (block.data.items, block.grad.items, block.classes.items, 0..) |_, grd, class, idx| {
        if (class != .wgt or grd == null) continue;
        f(ctx, graph, Tensor{ .ptr = graph, .class = .wgt, .idx = idx });
    }
    core.utils.synchronize_stream(graph.stream);
}

pub const SGD = struct {
    rate: f64,
    clip: ClipRange,

    pub fn init(config: struct { rate: f64, clip: ?ClipRange = null }) SGD {
        return .{ .rate = config.rate, .clip = config.clip orelse ClipRange.init() };
    }

    // w -= rate * clamp(g, lower, upper)
    pub fn update(self: *SGD, graph: *Graph) void {
        for_each_weight(graph, self, struct {
            fn apply(opt: *SGD, _: *Graph, w: Tensor) void {
                core.invoke(core.kernels.sgd, core.dkey(w), .{
                    w.data_ptr(), w.grad_ptr(), opt.rate, opt.clip.lower, opt.clip.upper, w.len(), w.context(),
                });
            }
        }.apply);
    }
};

pub const Momentum = struct {
    rate: f64,
    alpha: f64 = 0.90,
    clip: ClipRange,
    state: std.AutoHashMap(StateKey, *anyopaque), // per (graph, weight): m, zero on first use (optimizer.zig:249-256)

    const StateKey = struct { graph: usize, idx: usize };

    pub fn init(allocator: std.mem.Allocator, config: struct { rate: f64, alpha: f64 = 0.90, clip: ?ClipRange = null }) Momentum {
        return .{ .rate = config.rate, .alpha = config.alpha, .clip = config.clip orelse ClipRange.init(),
                  .state = std.AutoHashMap(StateKey, *anyopaque).init(allocator) };
    }

    fn slot(self: *Momentum, graph: *Graph, w: Tensor) *anyopaque {
        const key = StateKey{ .graph = @intFromPtr(graph), .idx = w.idx };
        if (self.state.get(key)) |m| return m;
        const m = graph.tensor_allocator.alloc(w.dtype(), w.len(), graph.stream);
        core.invoke(core.kernels.fill, core.dkey(w), .{ m, 0.0, w.len(), w.context() });
        self.state.put(key, m) catch @panic("out of memory");
        return m;
    }

    // m = alpha * m + clamp(g); w -= rate * m
    pub fn update(self: *Momentum, graph: *Graph) void {
        for_each_weight(graph, self, struct {
            fn apply(opt: *Momentum, g: *Graph, w: Tensor) void {
                core.invoke(core.kernels.momentum, core.dkey(w), .{
                    w.data_ptr(), w.grad_ptr(), opt.slot(g, w), opt.rate, opt.alpha, opt.clip.lower, opt.clip.upper, w.len(), w.context(),
                });
            }
        }.apply);
    }
};

pub const Adam = struct {
    rate: f64,
    beta1: f64 = 0.9,
    beta2: f64 = 0.999,
    eps: f64 = 1e-8,
    grad_scale: f64 = 1.0, // 1 / world_size after a summing all-reduce
    step: usize = 0,
    state: std.AutoHashMap(StateKey, Moments),

    const StateKey = struct { graph: usize, idx: usize };
    const Moments = struct { m: *anyopaque, v: *anyopaque };

    pub fn init(allocator: std.mem.Allocator, config: struct { rate: f64, beta1: f64 = 0.9, beta2: f64 = 0.999, eps: f64 = 1e-8 }) Adam {
        return .{ .rate = config.rate, .beta1 = config.beta1, .beta2 = config.beta2, .eps = config.eps,
                  .state = std.AutoHashMap(StateKey, Moments).init(allocator) };
    }

    fn slot(self: *Adam, graph: *Graph, w: Tensor) Moments {
        const key = StateKey{ .graph = @intFromPtr(graph), .idx = w.idx };
        if (self.state.get(key)) |mv| return mv;
        const mv = Moments{
            .m = graph.tensor_allocator.alloc(w.dtype(), w.len(), graph.stream),
            .v = graph.tensor_allocator.alloc(w.dtype(), w.len(), graph.stream),
        };
        core.invoke(core.kernels.fill, core.dkey(w), .{ mv.m, 0.0, w.len(), w.context() });
        core.invoke(core.kernels.fill, core.dkey(w), .{ mv.v, 0.0, w.len(), w.context() });
        self.state.put(key, mv) catch @panic("out of memory");
        return mv;
    }

    pub fn update(self: *Adam, graph: *Graph) void {
        self.step += 1;
        for_each_weight(graph, self, struct {
            fn apply(opt: *Adam, g: *Graph, w: Tensor) void {
                const mv = opt.slot(g, w);
                core.invoke(core.kernels.adam, core.dkey(w), .{
                    w.data_ptr(), w.grad_ptr(), mv.m, mv.v, opt.rate, opt.beta1, opt.beta2, opt.eps, opt.grad_scale, opt.step, w.len(), w.context(),
                });
            }
        }.apply);
    }
};
