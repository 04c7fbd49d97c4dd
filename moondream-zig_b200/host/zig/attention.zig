//! Replaces src/core/attention.zig: the three SDPA variants and the mask builder with the reference's
//! signatures, computed by the fused attention kernels (md_sdpa_maskless / _masked / _single).
const std = @import("std");
const Tensor = @import("../core/tensor.zig").Tensor;
const Allocator = std.mem.Allocator;
const cuda = @import("cuda_backend.zig");

const MAX_KV_LEN: usize = 2048; // attention.zig:252

/// softmax(Q K^T / sqrt(d)) V per head, no mask (attention.zig:125-234).
pub fn multiMasklessSDPA(
    n_heads: comptime_int,
    head_dim: comptime_int,
    query: Tensor(f16),
    key: Tensor(f16),
    value: Tensor(f16),
    allocator: Allocator,
) !Tensor(f16) {
    const q_len = query.shape[1];
    const kv_len = key.shape[1];
    var out = try Tensor(f16).init(allocator, &[_]usize{ n_heads, q_len, head_dim });
    errdefer out.deinit();
    try cuda.check(cuda.md_sdpa_maskless(try cuda.ctx(), cuda.h(query), cuda.h(key), cuda.h(value), cuda.hm(out), n_heads, q_len, kv_len, head_dim));
    return out;
}

/// [seq_len, pos + seq_len]: columns < pos all true, then lower-triangular (attention.zig:256-281).
pub fn createAttentionMask(allocator: Allocator, pos: usize, seq_len: usize) !Tensor(bool) {
    var mask = try Tensor(bool).init(allocator, &[_]usize{ seq_len, pos + seq_len });
    errdefer mask.deinit();
    // a Zig bool is one byte holding 0 or 1, which is what the kernel writes
    try cuda.check(cuda.md_create_attention_mask(try cuda.ctx(), @ptrCast(mask.data.ptr), pos, seq_len));
    return mask;
}

/// The same with a bool mask, false -> -inf before the softmax (attention.zig:416-541).
pub fn multiMaskedSDPA(
    query: Tensor(f16),
    key: Tensor(f16),
    value: Tensor(f16),
    mask: Tensor(bool),
    n_heads: usize,
    head_dim: usize,
    allocator: Allocator,
) !Tensor(f16) {
    const q_len = query.shape[1];
    const kv_len = key.shape[1];
    var out = try Tensor(f16).init(allocator, &[_]usize{ n_heads, q_len, head_dim });
    errdefer out.deinit();
    try cuda.check(cuda.md_sdpa_masked(try cuda.ctx(), cuda.h(query), cuda.h(key), cuda.h(value), @ptrCast(mask.data.ptr), cuda.hm(out), n_heads, q_len, kv_len, head_dim));
    return out;
}

/// One query token of 32 heads x 64 dims against the cache (attention.zig:759-811).
pub fn singleMaskedSDPA(
    query: Tensor(f16),
    key: Tensor(f16),
    value: Tensor(f16),
    mask: Tensor(bool),
    allocator: Allocator,
) !Tensor(f16) {
    const kv_len = key.shape[1];
    if (kv_len > MAX_KV_LEN) return error.SequenceTooLong;
    var out = try Tensor(f16).init(allocator, &[_]usize{ 32, 1, 64 });
    errdefer out.deinit();
    try cuda.check(cuda.md_sdpa_single(try cuda.ctx(), cuda.h(query), cuda.h(key), cuda.h(value), @ptrCast(mask.data.ptr), cuda.hm(out), kv_len));
    return out;
}

/// The reference frees its global thread pool here (attention.zig:814); the GPU path has none.
pub fn cleanupThreadPool() void {}
