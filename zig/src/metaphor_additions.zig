// Lines to merge into src/metaphor.zig (the facade, :13-56).  The README writes several names differently from
// the code (README.md:35,59-60,72,78-97 against metaphor.zig:20-56 and graph.zig:500-507); both spellings are
// exported, so the README's programs and the examples under src/examples compile against the same facade.
const core = @import("core");

pub const ops_additions = struct {
    pub const selu = @import("ops/selu.zig").forward;
    pub const linear = @import("ops/linear.zig").forward;
    pub const softmax = @import("ops/softmax.zig").forward;
    pub const rmsnorm = @import("ops/rmsnorm.zig").forward;
    pub const ssd_scan = @import("ops/ssd.zig").forward;
    pub const gated_norm = @import("ops/gated_norm.zig").forward;
    pub const permutate = @import("ops/permutate.zig").forward; // replaces the rank-2-only version
    pub const contraction = @import("ops/contraction.zig").forward; // rank-N "abc,cd->abd" through one (batched) launch
    pub const contractionScaled = @import("ops/contraction.zig").forward_scaled;
    // README spellings
    pub const innerProduct = @import("ops/inner_product.zig").forward;
    pub const innerProductScaled = @import("ops/inner_product.zig").forward_scaled;
};

pub const mem = struct { // README: mp.mem.fill; code: mp.algo.fill
    const impl = @import("algo/mem.zig");
    pub const fill = impl.fill;
    pub const copy = impl.copy;
    pub const sequence = impl.sequence;
};

pub const streams = struct { // README: mp.streams.synchronize; code: mp.stream.sync
    pub const init = core.utils.init_stream;
    pub const deinit = core.utils.deinit_stream;
    pub const synchronize = core.utils.synchronize_stream;
};

pub const optm = struct {
    const impl = @import("optm/optimizer.zig");
    pub const SGD = impl.SGD;
    pub const Momentum = impl.Momentum;
    pub const Adam = impl.Adam;
    pub const ClipRange = impl.ClipRange;
};
