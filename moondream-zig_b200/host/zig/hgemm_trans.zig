//! Replaces src/core/hgemm_trans.zig: same `matmul` (B given transposed, [N,K]), computed by md_hgemm_nt,
//! which takes the weight-streaming GEMV kernel for M <= 8 and the tcgen05 GEMM otherwise.
const std = @import("std");
const Allocator = std.mem.Allocator;
const Tensor = @import("../core/tensor.zig").Tensor;
const cuda = @import("cuda_backend.zig");

/// C[M,N] = A[M,K] . B_t[N,K]^T (hgemm_trans.zig:400-488).
pub fn matmul(a: Tensor(f16), b_transposed: Tensor(f16), allocator: Allocator) !Tensor(f16) {
    const A_shape = a.shape;
    const B_t_shape = b_transposed.shape;
    if (A_shape.len != 2 or B_t_shape.len != 2) {
        return error.InvalidTensorDimension;
    }
    const M = A_shape[0];
    const K = A_shape[1];
    const N = B_t_shape[0];
    if (B_t_shape[1] != K) {
        return error.IncompatibleTensorShapes;
    }
    var result = try Tensor(f16).initWithoutMemset(allocator, &[_]usize{ M, N });
    errdefer result.deinit();
    try cuda.check(cuda.md_hgemm_nt(try cuda.ctx(), cuda.h(a), cuda.h(b_transposed), cuda.hm(result), M, N, K));
    return result;
}
