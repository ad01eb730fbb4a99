// Replacement for `enable_gradient` of src/core/graph.zig:710-722.
//
// The reference allocates a gradient buffer the first time an op's reverse asks for it and then
// accumulates into it (`g_x = g_z + g_x`, `c += a*b`, GEMM with beta = 1) without ever
// initialising it: the first accumulation adds into whatever the allocator handed back.  The
// contract of this library is "gradient = 0 + sum of contributions", so the buffer is
// zero-filled on the graph's stream when it is created.
const core = @import("core");
const Tensor = core.Tensor;

pub fn enable_gradient(t: Tensor) void {
    const self = t.ptr;

    const grad_array = if (t.class == .hid)
        &self.node_block.grad
    else
        &self.leaf_block.grad;

    const grd = &grad_array.items[t.idx];

    if (grd.* == null) {
        grd.* = self.tensor_allocator.alloc(t.dtype(), t.len(), self.stream);
        core.invoke(core.kernels.fill, core.dkey(t), .{
            t.grad_ptr(),
            0.0,
            t.len(),
            t.context(),
        });
    }
}
