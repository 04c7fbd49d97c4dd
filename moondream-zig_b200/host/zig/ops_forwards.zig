//! Bodies for the four glue functions of src/core/ops.zig that sit between the GEMMs (the rest of ops.zig
//! is not on the hot path and stays as it is).  Paste each over the function of the same name.
const std = @import("std");
const Tensor = @import("tensor.zig").Tensor;
const cuda = @import("cuda_backend.zig");

/// ops.zig:312-323.
pub fn add(comptime T: type, tensor: *Tensor(T), other: Tensor(T)) !void {
    if (!std.mem.eql(usize, tensor.shape, other.shape)) {
        return error.ShapeMismatch;
    }
    if (T != f16) @compileError("the CUDA add is f16, the only type the models use");
    try cuda.check(cuda.md_add(try cuda.ctx(), cuda.hm(tensor.*), cuda.h(other), tensor.data.len));
}

/// ops.zig:1063-1070: normalises over the last dim; eps travels as its f16 bits.
pub fn layerNorm(comptime T: type, input: Tensor(T), weight: Tensor(T), bias: Tensor(T), eps: T) !Tensor(T) {
    if (T != f16) @compileError("the CUDA layerNorm is f16, the only type the models use");
    const cols = input.shape[input.shape.len - 1];
    if (weight.data.len != cols or bias.data.len != cols) return error.InvalidShape;
    const rows = input.data.len / cols;
    var out = try Tensor(T).init(input.allocator, input.shape);
    errdefer out.deinit();
    const eps_bits: u16 = @bitCast(eps);
    try cuda.check(cuda.md_layernorm(try cuda.ctx(), cuda.h(input), cuda.h(weight), cuda.h(bias), cuda.hm(out), rows, cols, eps_bits));
    return out;
}

/// ops.zig:1635-1774, in place.
pub fn gelu(comptime T: type, tensor: *Tensor(T)) !void {
    if (@typeInfo(T) != .Float) {
        @compileError("GELU operation requires floating-point tensor");
    }
    if (T != f16) @compileError("the CUDA gelu is f16, the only type the models use");
    try cuda.check(cuda.md_gelu(try cuda.ctx(), cuda.hm(tensor.*), tensor.data.len));
}

/// ops.zig:1780-1953: a += b broadcast over the leading dims of a.  The models' uses are a bias [cols] on
/// [rows, cols] and the position embedding [1, 729, 1152] on [crops, 729, 1152]: in both b is a whole
/// trailing block of a, which is what the kernel repeats.
pub fn broadcast_add_simd(a: *Tensor(f16), b: Tensor(f16)) !void {
    if (b.shape.len > a.shape.len) {
        return error.InvalidBroadcast;
    }
    var leading_ones = true;
    for (0..b.shape.len) |i| {
        const a_dim = a.shape[a.shape.len - 1 - i];
        const b_dim = b.shape[b.shape.len - 1 - i];
        if (b_dim != a_dim and b_dim != 1) {
            return error.IncompatibleBroadcast;
        }
    }
    // inner dims of size 1 (other than leading ones) are not a trailing block
    for (0..b.shape.len) |i| {
        const b_dim = b.shape[i];
        const a_dim = a.shape[a.shape.len - b.shape.len + i];
        if (b_dim == 1 and a_dim != 1) {
            if (!leading_ones) return error.IncompatibleBroadcast;
        } else {
            leading_ones = false;
        }
    }
    const block = b.data.len;
    if (block == 0 or a.data.len % block != 0) return error.IncompatibleBroadcast;
    try cuda.check(cuda.md_bias_add(try cuda.ctx(), cuda.hm(a.*), cuda.h(b), a.data.len / block, block));
}
