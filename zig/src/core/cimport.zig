// Replaces the generated src/core/cimport.zig (file_gen.zig:330-340): the three headers of the
// reference's device layer become the headers of this library.  MP_INCLUDE_DIR is the `include/`
// directory of this repository, passed by build.zig with `addIncludePath`.
pub const C = @cImport({
    @cInclude("mp_types.h");
    @cInclude("mp_device_utils.h");
    @cInclude("mp_kernels.h");
    @cInclude("mp_jit.h");
    @cInclude("mp_comm.h");
});
