//! Binding of libmoondream_b200 (include/moondream_b200.h) for the Zig 0.13 host of moondream-zig.
//! Copy this directory's files over the reference's src/core/ files of the same name (hgemm.zig,
//! hgemm_trans.zig, attention.zig, rope.zig), put cuda_backend.zig next to them, paste the bodies of
//! ops_forwards.zig / sampling_forwards.zig over the functions of the same name in src/core/ops.zig and
//! src/utils/sampling.zig, and apply build_cuda.zig.patch to build.zig.  Every `pub fn` keeps the name,
//! the parameter list and the error behaviour of the function it replaces, so src/model/*.zig and
//! src/moondream.zig compile unchanged.
//!
//! One context per process (the reference is single-threaded at these call sites, text_model.zig:139-345).
//! Tensors stay host tensors owned by the caller's allocator; every call stages its operands through
//! device memory and returns when the result is back (drop-in mode).  Weights registered with
//! uploadWeight live on the device for the whole process and may be passed wherever a `b` operand goes.
const std = @import("std");
const Tensor = @import("tensor.zig").Tensor;

pub const MdStatus = enum(c_int) {
    ok = 0,
    invalid_arg = 1,
    invalid_dimension = 2,
    shape = 3,
    sequence_too_long = 4,
    invalid_rot_dim = 5,
    unsupported = 6,
    oom = 7,
    cuda = 8,
    timeout = 9,
    no_device = 10,
    io = 11,
    format = 12,
    nccl = 13,
    _,
};

pub const MdCtx = opaque {};

pub extern fn md_init(out: *?*MdCtx, device: c_int) c_int;
pub extern fn md_destroy(ctx: ?*MdCtx) c_int;
pub extern fn md_last_error(ctx: ?*const MdCtx) [*:0]const u8;
pub extern fn md_sync(ctx: ?*MdCtx) c_int;
pub extern fn md_upload(ctx: ?*MdCtx, host: *const anyopaque, bytes: usize, dev_out: *?*anyopaque) c_int;
pub extern fn md_free(ctx: ?*MdCtx, dev: ?*anyopaque) c_int;
pub extern fn md_hgemm_nn(ctx: ?*MdCtx, a: [*]const u16, b: [*]const u16, c: [*]u16, M: usize, N: usize, K: usize) c_int;
pub extern fn md_hgemm_nt(ctx: ?*MdCtx, a: [*]const u16, b_t: [*]const u16, c: [*]u16, M: usize, N: usize, K: usize) c_int;
pub extern fn md_sdpa_maskless(ctx: ?*MdCtx, q: [*]const u16, k: [*]const u16, v: [*]const u16, out: [*]u16, n_heads: usize, q_len: usize, kv_len: usize, head_dim: usize) c_int;
pub extern fn md_create_attention_mask(ctx: ?*MdCtx, mask: [*]u8, pos: usize, seq_len: usize) c_int;
pub extern fn md_sdpa_masked(ctx: ?*MdCtx, q: [*]const u16, k: [*]const u16, v: [*]const u16, mask: [*]const u8, out: [*]u16, n_heads: usize, q_len: usize, kv_len: usize, head_dim: usize) c_int;
pub extern fn md_sdpa_single(ctx: ?*MdCtx, q: [*]const u16, k: [*]const u16, v: [*]const u16, mask: [*]const u8, out: [*]u16, kv_len: usize) c_int;
pub extern fn md_rope_table(ctx: ?*MdCtx, table: [*]f32, dim: usize, end: usize, theta: f32) c_int;
pub extern fn md_rope_apply(ctx: ?*MdCtx, x: [*]const u16, out: [*]u16, n_heads: usize, seq_len: usize, head_dim: usize, freqs_cis: [*]const f32, freqs_half: usize, position_ids: [*]const u64, rot_dim: usize) c_int;
pub extern fn md_layernorm(ctx: ?*MdCtx, x: [*]const u16, w: [*]const u16, b: [*]const u16, y: [*]u16, rows: usize, cols: usize, eps_f16: u16) c_int;
pub extern fn md_gelu(ctx: ?*MdCtx, x: [*]u16, n: usize) c_int;
pub extern fn md_bias_add(ctx: ?*MdCtx, a: [*]u16, b: [*]const u16, rows: usize, cols: usize) c_int;
pub extern fn md_add(ctx: ?*MdCtx, a: [*]u16, b: [*]const u16, n: usize) c_int;
pub extern fn md_argmax(ctx: ?*MdCtx, x: [*]const u16, n: usize, idx_out: *u64) c_int;

var the_ctx: ?*MdCtx = null;

/// The process-wide context, created on first use on device MOONDREAM_DEVICE (default 0).
/// There is no CPU fallback: without an sm_100a device this returns error.NoCudaDevice.
pub fn ctx() !*MdCtx {
    if (the_ctx) |c| return c;
    var device: c_int = 0;
    if (std.posix.getenv("MOONDREAM_DEVICE")) |s| device = std.fmt.parseInt(c_int, s, 10) catch 0;
    var out: ?*MdCtx = null;
    const st = md_init(&out, device);
    if (st != 0 or out == null) {
        std.log.err("moondream_b200: {s}", .{md_last_error(null)});
        return error.NoCudaDevice;
    }
    the_ctx = out;
    return out.?;
}

pub fn deinit() void {
    if (the_ctx) |c| _ = md_destroy(c);
    the_ctx = null;
}

/// md_status -> the Zig error the replaced function would have returned.
pub fn check(status: c_int) !void {
    const st: MdStatus = @enumFromInt(status);
    return switch (st) {
        .ok => {},
        .invalid_dimension => error.InvalidTensorDimension,
        .shape => error.IncompatibleTensorShapes,
        .sequence_too_long => error.SequenceTooLong,
        .invalid_rot_dim => error.InvalidRotationDimension,
        .oom => error.OutOfMemory,
        else => blk: {
            std.log.err("moondream_b200: {s}", .{md_last_error(the_ctx)});
            break :blk error.CudaFailure;
        },
    };
}

pub fn h(t: Tensor(f16)) [*]const u16 {
    return @ptrCast(t.data.ptr);
}

pub fn hm(t: Tensor(f16)) [*]u16 {
    return @ptrCast(t.data.ptr);
}

/// Weights live for the whole process (preslice_text.zig:53-79): upload once and keep the device pointer.
/// Never key a cache on the host address: the slab allocator recycles addresses
/// (slab_reusing_allocator.zig:141-156).
pub fn uploadWeight(t: Tensor(f16)) ![*]const u16 {
    var dev: ?*anyopaque = null;
    try check(md_upload(try ctx(), @ptrCast(t.data.ptr), t.data.len * @sizeOf(f16), &dev));
    return @ptrCast(@alignCast(dev.?));
}
