//! Body for `argmax` of src/utils/sampling.zig (the greedy sampling of moondream.zig:335-337).
const std = @import("std");
const Tensor = @import("../core/tensor.zig").Tensor;
const cuda = @import("../core/cuda_backend.zig");

/// First index of the strict maximum (sampling.zig:257-273).
pub fn argmax(comptime T: type, tensor: *const Tensor(T)) !usize {
    if (tensor.data.len == 0) {
        return error.EmptyTensor;
    }
    if (T != f16) @compileError("the CUDA argmax is f16, the only type the models use");
    var idx: u64 = 0;
    try cuda.check(cuda.md_argmax(try cuda.ctx(), cuda.h(tensor.*), tensor.data.len, &idx));
    return @intCast(idx);
}
