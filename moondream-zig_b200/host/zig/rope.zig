//! Replaces src/core/rope.zig: frequency table and rotary embedding with the reference's signatures.
const std = @import("std");
const Tensor = @import("../core/tensor.zig").Tensor;
const Allocator = std.mem.Allocator;
const cuda = @import("cuda_backend.zig");

const FreqsError = error{
    DimensionTooSmall,
    DimensionNotEven,
    EndTooSmall,
    ThetaTooSmall,
    InvalidShape,
    ComputationOverflow,
    NumericalInstability,
    OutOfMemory,
    CudaFailure,
};

/// (cos, sin) of p * theta^(-2j/dim), shape [end, dim/2, 2] (rope.zig:32-128).  The table is computed on the
/// device in f32 and copied back; the reference's caller uses T = f32 (text_model.zig:88).
pub fn precomputeFreqsCis(
    comptime T: type,
    allocator: std.mem.Allocator,
    dim: usize,
    end: usize,
    theta: T,
) FreqsError!Tensor(T) {
    if (dim <= 0) return error.DimensionTooSmall;
    if (dim % 2 != 0) return error.DimensionNotEven;
    if (end <= 0) return error.EndTooSmall;
    if (theta <= 0) return error.ThetaTooSmall;
    if (T != f32) @compileError("the CUDA rope table is f32, as the reference's only caller asks for");
    var table = Tensor(T).init(allocator, &[_]usize{ end, dim / 2, 2 }) catch return error.OutOfMemory;
    errdefer table.deinit();
    const c = cuda.ctx() catch return error.CudaFailure;
    if (cuda.md_rope_table(c, @ptrCast(table.data.ptr), dim, end, theta) != 0) return error.CudaFailure;
    return table;
}

/// Rotates the first rot_dim dims of every head, pairs (j, j + rot_dim/2) (rope.zig:130-272).
pub fn applyRotEmb(
    allocator: Allocator,
    x: Tensor(f16),
    n_heads: usize,
    head_dim: usize,
    freqs_cis: Tensor(f32),
    position_ids: Tensor(usize),
    rot_dim: usize,
) !Tensor(f16) {
    if (x.shape.len != 3) return error.InvalidInputDimensions;
    if (rot_dim != freqs_cis.shape[freqs_cis.shape.len - 2] * 2) {
        return error.InvalidRotationDimension;
    }
    const seq_len = x.shape[1];
    var out = try Tensor(f16).init(allocator, x.shape);
    errdefer out.deinit();
    try cuda.check(cuda.md_rope_apply(try cuda.ctx(), cuda.h(x), cuda.hm(out), n_heads, seq_len, head_dim, @ptrCast(freqs_cis.data.ptr), rot_dim / 2, @ptrCast(position_ids.data.ptr), rot_dim));
    return out;
}
