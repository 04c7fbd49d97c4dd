//! Replaces src/core/hgemm.zig: same `matmul`, computed by md_hgemm_nn on the B200.
const std = @import("std");
const Allocator = std.mem.Allocator;
const Tensor = @import("tensor.zig").Tensor;
const cuda = @import("cuda_backend.zig");

/// C[M,N] = A[M,K] . B[K,N], f16 in and out, f32 accumulation, one rounding (hgemm.zig:362-426).
pub fn matmul(a: Tensor(f16), b: Tensor(f16), allocator: Allocator) !Tensor(f16) {
    const A_shape = a.shape;
    const B_shape = b.shape;
    if (A_shape.len != 2 or B_shape.len != 2) {
        return error.InvalidTensorDimension;
    }
    const M = A_shape[0];
    const K = A_shape[1];
    const N = B_shape[1];
    if (B_shape[0] != K) {
        return error.IncompatibleTensorShapes;
    }
    var result = try Tensor(f16).initWithoutMemset(allocator, &[_]usize{ M, N });
    errdefer result.deinit();
    try cuda.check(cuda.md_hgemm_nn(try cuda.ctx(), cuda.h(a), cuda.h(b), cuda.hm(result), M, N, K));
    return result;
}
