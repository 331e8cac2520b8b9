//! Drop-in `CudaDevice` for zigrad on top of the B200 library (libamalgamate.so).
//!
//! Replaces `src/device/cuda_device.zig` of the reference.  It binds the same
//! headers through `src/cuda/root.zig` (`@cImport` of decls.h, cuda_utils.h,
//! blas_conflux.h, nn_conflux.h) plus `zg_b200.h`, keeps the method-per-opspec
//! shape that `DeviceReference.dispatch` discovers with `@hasDecl`
//! (`src/device/device_reference.zig:15-27`), and panics where the reference
//! library exits the process.
//!
//! NOT COMPILED in this repository: the build image has no Zig toolchain.  The
//! C ABI underneath is exercised by the Python twin of this file
//! (zigrad_b200/device.py) in the GPU tests.
const std = @import("std");
const cuda = @import("cuda"); // src/cuda/root.zig + `@cInclude("zg_b200.h")`
const opspec = @import("opspec.zig");
const DeviceData = @import("../allocators.zig").DeviceData;
const Error = @import("../allocators.zig").Error;
const TransferDirection = @import("device_common.zig").TransferDirection;
const RandType = @import("device_common.zig").RandType;

const Self = @This();
pub const DeviceReference = @import("device_reference.zig");

context: struct {
    device_number: u32,
    properties: cuda.DevicePropertiesWrapper,
    stream: cuda.StreamWrapper,
    cublas: cuda.CublasWrapper, // stream-bound op contexts; no vendor library behind them
    cudnn: cuda.CudnnWrapper,
    cutensor: cuda.CutensorWrapper,
},
cache: cuda.CacheWrapper, // stream-ordered cache inside the library (replaces CachingAllocator(DataHandler))
capture: ExecutionGraph,

pub fn device_count() u32 {
    return cuda.device_count();
}

pub fn init(device_number: u32) Self {
    const properties = cuda.init_device(device_number);
    const stream = cuda.init_stream();
    var self: Self = .{
        .context = .{
            .device_number = device_number,
            .properties = properties,
            .stream = stream,
            .cublas = cuda.init_cublas_handle(stream),
            .cudnn = cuda.init_cudnn_handle(stream),
            .cutensor = cuda.init_cutensor_handle(stream),
        },
        .cache = cuda.zg_cache_create(device_number, 0),
        .capture = .{},
    };
    self.check();
    return self;
}

pub fn deinit(self: *Self) void {
    self.sync();
    self.capture.free(self);
    cuda.zg_cache_destroy(self.cache);
    cuda.deinit_cudnn_handle(self.context.cudnn);
    cuda.deinit_cublas_handle(self.context.cublas);
    cuda.deinit_cutensor_handle(self.context.cutensor);
    cuda.deinit_stream(self.context.stream);
    self.* = undefined;
}

pub fn reference(self: *Self) DeviceReference {
    return .{ .ptrs = .{ .cuda = self } };
}

/// The reference library prints and exits on a CUDA error; this one records a
/// sticky status, which becomes a panic here (same observable contract).
fn check(_: *const Self) void {
    if (cuda.zg_last_error() != 0) @panic(std.mem.span(cuda.zg_last_error_message()));
}

pub fn dtype(T: type) cuda.dtype {
    return switch (T) {
        f32 => cuda.SINGLE,
        f64 => cuda.DOUBLE,
        else => @panic("Only supports floating point, found: " ++ @typeName(T)),
    };
}

// ---------------------------------------------------------------- element wise
pub fn add(self: *const Self, T: type, p: opspec.add(T)) void {
    cuda.addition(dtype(T), self.context.stream, p.x.ptr, p.y.ptr, p.z.ptr, p.x.len, p.y.len, p.z.len);
}
pub fn sub(self: *const Self, T: type, p: opspec.sub(T)) void {
    cuda.subtraction(dtype(T), self.context.stream, p.x.ptr, p.y.ptr, p.z.ptr, p.x.len, p.y.len, p.z.len);
}
pub fn mul(self: *const Self, T: type, p: opspec.mul(T)) void {
    cuda.multiplication(dtype(T), self.context.stream, p.x.ptr, p.y.ptr, p.z.ptr, p.x.len, p.y.len, p.z.len);
}
pub fn div(self: *const Self, T: type, p: opspec.div(T)) void {
    cuda.division(dtype(T), self.context.stream, p.x.ptr, p.y.ptr, p.z.ptr, p.x.len, p.y.len, p.z.len);
}

// -------------------------------------------------------------- linear algebra
pub fn dot(self: *const Self, T: type, p: opspec.dot(T)) void {
    cuda.dot(dtype(T), self.context.cublas, p.x.ptr, p.y.ptr, p.z.ptr, p.x.len);
}
pub fn axpy(self: *const Self, T: type, p: opspec.axpy(T)) void {
    // alpha may point to host memory (SGD) or device memory (dot backward); the library inspects it
    cuda.axpy(dtype(T), self.context.cublas, p.x.ptr, p.y.ptr, p.x.len, p.alpha);
}
pub fn outer(self: *const Self, T: type, p: opspec.outer(T)) void {
    cuda.ger(dtype(T), self.context.cublas, p.x.ptr, p.y.ptr, p.A.ptr, p.x.len, p.y.len, p.y.len, p.alpha);
}
pub fn transpose(self: *const Self, T: type, p: opspec.transpose(T)) void {
    cuda.zg_transpose(dtype(T), self.context.stream, p.A.ptr, p.B.ptr, p.m, p.n, p.alpha);
}
pub fn matvec(self: *const Self, T: type, p: opspec.matvec(T)) void {
    cuda.gemv(dtype(T), self.context.cublas, p.A.ptr, p.x.ptr, p.y.ptr, p.m, p.n, p.trans_a, p.alpha, p.beta);
}
pub fn matmul(self: *const Self, T: type, p: opspec.matmul(T)) void {
    cuda.gemm(dtype(T), self.context.cublas, p.A.ptr, p.B.ptr, p.C.ptr, p.m, p.n, p.k, p.trans_a, p.trans_b, p.lda, p.ldb, p.ldc, p.alpha, p.beta);
}
pub fn bmm_acc(self: *const Self, T: type, p: opspec.bmm_acc(T)) void {
    // shapes are {batch, M, K}, {batch, K, N}, {batch, M, N} (src/ndarray.zig:881-895)
    cuda.zg_bmm(
        dtype(T),       dtype(T),       self.context.stream,
        p.A.ptr,        p.B.ptr,        p.C.ptr,
        p.A_shape[0],   p.B_shape[0],   p.C_shape[0],
        p.C_shape[1],   p.C_shape[2],   p.A_shape[2],
        p.trans_a,      p.trans_b,      p.lda,
        p.ldb,          p.ldc,          p.alpha,
        p.beta,         cuda.ZG_EPI_NONE, null,
        null,           null,
    );
}
pub fn sum(self: *const Self, T: type, p: opspec.sum(T)) void {
    cuda.reduce_sum(dtype(T), self.context.cublas, p.x.ptr, p.y.ptr, p.x.len);
}
pub fn scale(self: *const Self, T: type, p: opspec.scale(T)) void {
    cuda.scale(dtype(T), self.context.cublas, p.x.ptr, p.x.len, p.alpha);
}
pub fn nrm2(self: *const Self, T: type, p: opspec.nrm2(T)) void {
    cuda.nrm2(dtype(T), self.context.cublas, p.x.ptr, p.y.ptr, p.x.len);
}
pub fn clip_nrm2(self: *Self, T: type, p: opspec.clip_nrm2(T)) void {
    const scratch = self.mem_scratch(T, 1);
    cuda.clip_nrm2(dtype(T), self.context.cublas, p.x.ptr, scratch.ptr, p.x.len, p.max_norm, p.delta);
}

// ------------------------------------------------------------------ non-linear
pub fn exp_fwd(self: *const Self, T: type, p: opspec.exp_fwd(T)) void {
    cuda.zg_unary_fwd(dtype(T), self.context.stream, cuda.ZG_UN_EXP, p.x.ptr, p.y.ptr, p.x.len, 0);
}
pub fn exp_bwd(self: *const Self, T: type, p: opspec.exp_bwd(T)) void {
    cuda.zg_unary_bwd(dtype(T), self.context.stream, cuda.ZG_UN_EXP, p.y.ptr, p.y_g.ptr, p.x_g.ptr, p.y.len, 0);
}
pub fn sqrt_fwd(self: *const Self, T: type, p: opspec.sqrt_fwd(T)) void {
    cuda.zg_unary_fwd(dtype(T), self.context.stream, cuda.ZG_UN_SQRT, p.x.ptr, p.y.ptr, p.x.len, 0);
}
pub fn sqrt_bwd(self: *const Self, T: type, p: opspec.sqrt_bwd(T)) void {
    cuda.zg_unary_bwd(dtype(T), self.context.stream, cuda.ZG_UN_SQRT, p.x.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len, p.eps);
}
pub fn rsqrt_fwd(self: *const Self, T: type, p: opspec.rsqrt_fwd(T)) void {
    cuda.zg_unary_fwd(dtype(T), self.context.stream, cuda.ZG_UN_RSQRT, p.x.ptr, p.y.ptr, p.x.len, p.eps);
}
pub fn rsqrt_bwd(self: *const Self, T: type, p: opspec.rsqrt_bwd(T)) void {
    cuda.zg_unary_bwd(dtype(T), self.context.stream, cuda.ZG_UN_RSQRT, p.x.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len, p.eps);
}
pub fn tanh_fwd(self: *const Self, T: type, p: opspec.tanh_fwd(T)) void {
    cuda.zg_unary_fwd(dtype(T), self.context.stream, cuda.ZG_UN_TANH, p.x.ptr, p.y.ptr, p.x.len, 0);
}
pub fn tanh_bwd(self: *const Self, T: type, p: opspec.tanh_bwd(T)) void {
    cuda.zg_unary_bwd(dtype(T), self.context.stream, cuda.ZG_UN_TANH, p.y.ptr, p.y_g.ptr, p.x_g.ptr, p.y.len, 0);
}
pub fn sigm_fwd(self: *const Self, T: type, p: opspec.sigm_fwd(T)) void {
    cuda.zg_unary_fwd(dtype(T), self.context.stream, cuda.ZG_UN_SIGM, p.x.ptr, p.y.ptr, p.x.len, 0);
}
pub fn sigm_bwd(self: *const Self, T: type, p: opspec.sigm_bwd(T)) void {
    cuda.zg_unary_bwd(dtype(T), self.context.stream, cuda.ZG_UN_SIGM, p.y.ptr, p.y_g.ptr, p.x_g.ptr, p.y.len, 0);
}
pub fn pow_fwd(self: *const Self, T: type, p: opspec.pow_fwd(T)) void {
    cuda.zg_unary_fwd(dtype(T), self.context.stream, cuda.ZG_UN_POW, p.x.ptr, p.y.ptr, p.x.len, p.exp);
}
pub fn pow_fwd_(self: *const Self, T: type, p: opspec.pow_fwd_(T)) void {
    cuda.zg_unary_fwd(dtype(T), self.context.stream, cuda.ZG_UN_POW, p.x.ptr, p.x.ptr, p.x.len, p.exp);
}
pub fn pow_bwd(self: *const Self, T: type, p: opspec.pow_bwd(T)) void {
    cuda.zg_pow_bwd(dtype(T), self.context.stream, p.x.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len, p.exp, p.eps);
}
pub fn sqrt_fwd_(self: *const Self, T: type, p: opspec.sqrt_fwd_(T)) void {
    cuda.zg_unary_fwd(dtype(T), self.context.stream, cuda.ZG_UN_SQRT, p.x.ptr, p.x.ptr, p.x.len, 0);
}
pub fn tanh_inplace_bwd(self: *const Self, T: type, p: opspec.tanh_inplace_bwd(T)) void {
    cuda.zg_unary_inplace_bwd(dtype(T), self.context.stream, cuda.ZG_UN_TANH, p.x.ptr, p.x_g.ptr, p.x.len);
}
pub fn sigm_inplace_bwd(self: *const Self, T: type, p: opspec.sigm_inplace_bwd(T)) void {
    cuda.zg_unary_inplace_bwd(dtype(T), self.context.stream, cuda.ZG_UN_SIGM, p.x.ptr, p.x_g.ptr, p.x.len);
}
pub fn relu_mask_fwd(self: *const Self, T: type, p: opspec.relu_mask_fwd(T)) void {
    cuda.zg_relu_mask_fwd(dtype(T), self.context.stream, p.x.ptr, p.mask.ptr, p.x.len);
}
pub fn relu_mask_bwd(self: *const Self, T: type, p: opspec.relu_mask_bwd(T)) void {
    cuda.zg_relu_mask_bwd(dtype(T), self.context.stream, p.x_g.ptr, p.mask.ptr, p.x_g.len);
}
pub fn clamp_mask_fwd(self: *const Self, T: type, p: opspec.clamp_mask_fwd(T)) void {
    cuda.zg_clamp_mask_fwd(dtype(T), self.context.stream, p.x.ptr, p.y.ptr, p.mask.ptr, p.x.len, p.min, p.max);
}
pub fn clamp_mask_bwd(self: *const Self, T: type, p: opspec.clamp_mask_bwd(T)) void {
    cuda.zg_clamp_mask_bwd(dtype(T), self.context.stream, p.x_g.ptr, p.y_g.ptr, p.mask.ptr, p.x_g.len);
}
pub fn relu_fwd(self: *const Self, T: type, p: opspec.relu_fwd(T)) void {
    cuda.relu_fwd(dtype(T), self.context.stream, p.x.ptr, p.y.ptr, p.x.len);
}
pub fn relu_bwd(self: *const Self, T: type, p: opspec.relu_bwd(T)) void {
    cuda.relu_bwd(dtype(T), self.context.stream, p.x.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len);
}
pub fn relu_inplace_bwd(self: *const Self, T: type, p: opspec.relu_inplace_bwd(T)) void {
    cuda.zg_relu_inplace_bwd(dtype(T), self.context.stream, p.x.ptr, p.x_g.ptr, p.x.len);
}
pub fn max_fwd(self: *const Self, T: type, p: opspec.max_fwd(T)) void {
    cuda.max_fwd(dtype(T), self.context.stream, p.x.ptr, p.y.ptr, p.x.len);
}
pub fn max_bwd(self: *const Self, T: type, p: opspec.max_bwd(T)) void {
    cuda.max_bwd(dtype(T), self.context.stream, p.x.ptr, p.y.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len);
}
pub fn clamp_fwd(self: *const Self, T: type, p: opspec.clamp_fwd(T)) void {
    cuda.clamp(dtype(T), self.context.stream, p.x.ptr, p.y.ptr, p.x.len, p.min, p.max);
}
pub fn clamp_bwd(self: *const Self, T: type, p: opspec.clamp_bwd(T)) void {
    cuda.zg_clamp_bwd(dtype(T), self.context.stream, p.x.ptr, p.y_g.ptr, p.x_g.ptr, p.x.len, p.min, p.max);
}

// ------------------------------------------------------------------ reductions
pub fn unbroadcast(self: *const Self, T: type, p: opspec.unbroadcast(T)) void {
    cuda.zg_unbroadcast(dtype(T), self.context.stream, p.x.ptr, p.x_shape.ptr, p.x_shape.len, p.y.ptr, p.y_shape.ptr, p.y_shape.len, p.scratch.ptr, p.alpha, p.beta);
}
pub fn broadcast(self: *const Self, T: type, p: opspec.broadcast(T)) void {
    cuda.zg_broadcast(dtype(T), self.context.stream, p.x.ptr, p.x.len, p.y.ptr, p.y.len, p.alpha, p.beta);
}
pub fn sum_along(self: *const Self, T: type, p: opspec.sum_along(T)) void {
    cuda.zg_sum_along(dtype(T), self.context.stream, p.x.ptr, p.x_shape.ptr, p.x_shape.len, p.dim, p.y.ptr, p.alpha, p.beta);
}
pub fn max_along(self: *const Self, T: type, p: opspec.max_along(T)) void {
    cuda.zg_max_along(dtype(T), self.context.stream, p.x.ptr, p.x_shape.ptr, p.x_shape.len, p.dim, p.y.ptr);
}

// ----------------------------------------------------------------------- index
pub fn scatter_add(self: *const Self, T: type, p: opspec.scatter_add(T)) void {
    cuda.zg_scatter_add(dtype(T), self.context.stream, p.src.ptr, p.offsets.ptr, p.src.len, p.dst.ptr);
}
pub fn scatter_add_2d(self: *const Self, T: type, p: opspec.scatter_add_2d(T)) void {
    cuda.zg_scatter_add_2d(dtype(T), self.context.stream, p.src.ptr, p.indices.ptr, p.indices.len, p.stride, p.dst.ptr);
}
pub fn scatter_add_csr(self: *const Self, T: type, p: opspec.scatter_add_csr(T)) void {
    cuda.zg_scatter_add_csr(dtype(T), self.context.stream, p.src.ptr, p.row_ptr.ptr, p.src.len, p.dst.ptr);
}
pub fn segment_sum_csr(self: *const Self, T: type, p: opspec.segment_sum_csr(T)) void {
    cuda.zg_segment_sum_csr(dtype(T), self.context.stream, p.src.ptr, p.row_offsets.ptr, p.dst.len, p.dst.ptr);
}
pub fn scatter_gcn_deg_scaled(self: *const Self, T: type, p: opspec.scatter_gcn_deg_scaled(T)) void {
    cuda.zg_scatter_gcn_deg_scaled(dtype(T), self.context.stream, p.dst.ptr, p.h.ptr, p.deg.ptr, p.src_indices.ptr, p.tgt_indices.ptr, p.stride, p.n_edge);
}
pub fn scatter_gcn_deg_scaled_bwd(self: *const Self, T: type, p: opspec.scatter_gcn_deg_scaled_bwd(T)) void {
    cuda.zg_scatter_gcn_deg_scaled_bwd(dtype(T), self.context.stream, p.grad_output.ptr, p.h.ptr, p.deg.ptr, p.src_indices.ptr, p.tgt_indices.ptr, p.grad_h.ptr, p.grad_deg.ptr, p.stride, p.n_edge);
}

// ------------------------------------------------------ ops added to the opspec
// (the struct definitions these methods take are additions to src/device/opspec.zig: softmax_ce, smooth_l1, sgd, adam, linear)
pub fn softmax_ce(self: *const Self, T: type, p: opspec.softmax_ce(T)) void {
    cuda.zg_softmax_ce_fwd_bwd(dtype(T), self.context.stream, p.logits.ptr, p.labels.ptr, cuda.ZG_LABEL_ONEHOT, p.rows, p.classes, p.ld, p.loss_div, p.loss.ptr, if (p.grad) |g| g.ptr else null, @intFromBool(p.accumulate), null, if (p.bias_grad) |b| b.ptr else null);
}
pub fn smooth_l1(self: *const Self, T: type, p: opspec.smooth_l1(T)) void {
    cuda.zg_smooth_l1_fwd_bwd(dtype(T), self.context.stream, p.pred.ptr, p.target.ptr, p.pred.len, p.beta, p.loss.ptr, if (p.grad) |g| g.ptr else null);
}
pub fn sgd(self: *const Self, T: type, p: opspec.sgd(T)) void {
    cuda.zg_sgd_step(dtype(T), self.context.stream, p.params.ptr, p.grads.ptr, p.segments.ptr, p.segments.len, p.lr, @intFromBool(p.clip), p.max_norm, p.delta, p.norms.ptr, @intFromBool(p.zero_grads));
}
pub fn adam(self: *const Self, T: type, p: opspec.adam(T)) void {
    cuda.zg_adam_step(dtype(T), self.context.stream, p.params.ptr, p.grads.ptr, p.m.ptr, p.v.ptr, p.segments.ptr, p.segments.len, p.t_first, p.lr, p.beta1, p.beta2, p.eps, @intFromBool(p.clip), p.max_norm, p.delta, p.norms.ptr, null, null);
}
pub fn linear(self: *const Self, T: type, p: opspec.linear(T)) void {
    if (p.sm_budget > 0) cuda.zg_bmm_sm_budget(p.sm_budget); // GEMMs side by side on parallel streams share the SMs
    cuda.zg_bmm(dtype(T), dtype(T), self.context.stream, p.A.ptr, p.B.ptr, p.C.ptr, 1, 1, 1, p.m, p.n, p.k, p.trans_a, p.trans_b, p.lda, p.ldb, p.ldc, p.alpha, p.beta, @intFromEnum(p.epilogue), if (p.bias) |b| b.ptr else null, if (p.mask_src) |m| m.ptr else null, if (p.colsum) |c| c.ptr else null);
}
/// The last two Linear layers, their softmax cross-entropy and the backward pass down to the gradient of the
/// layer in front of them as one kernel (the separate ops when `mlp_tail_supported` says no).
pub fn mlp_tail_supported(_: *const Self, T: type, h1: usize, h2: usize, classes: usize) bool {
    return cuda.zg_mlp_tail_supported(dtype(T), h1, h2, classes) != 0;
}
pub fn mlp_tail(self: *const Self, T: type, p: opspec.mlp_tail(T)) void {
    const labels: ?*const anyopaque = if (p.label_index) |l| @ptrCast(l.ptr) else @ptrCast(p.onehot.?.ptr);
    cuda.zg_mlp_tail_fwd_bwd(dtype(T), self.context.stream, p.rows, p.h1, p.h2, p.classes, p.act0.ptr, p.W1.ptr, p.b1.ptr, p.W2.ptr, p.b2.ptr, labels, if (p.label_index != null) cuda.ZG_LABEL_INDEX else cuda.ZG_LABEL_ONEHOT, p.ld_out, p.loss_div, p.act1.ptr, p.logits.ptr, p.loss.ptr, p.dlogits.ptr, p.dact1.ptr, p.dact0.ptr, p.db2.ptr, p.db1.ptr, p.db0.ptr, @intFromBool(p.weights_ready));
}
pub fn sm_count(_: *const Self) usize {
    return @intCast(cuda.zg_sm_count());
}

// ----------------------------------------------------------------- collectives
/// Library collectives (NCCL bound at run time).  Rank 0 fills a 128-byte id with `comm_unique_id` and hands it to the
/// other ranks over any host channel; every rank then calls `comm_init`.
pub const Communicator = cuda.CommWrapper;
pub fn comm_unique_id(id: *[128]u8) void {
    cuda.zg_nccl_unique_id(id);
}
pub fn comm_init(self: *const Self, id: *const [128]u8, rank: u32, world: u32) error{CommInitFailed}!Communicator {
    const c = cuda.zg_comm_init_rank(id, rank, world);
    self.check();
    if (c.ptr == null) return error.CommInitFailed;
    return c;
}
pub fn comm_deinit(_: *const Self, comm: Communicator) void {
    cuda.zg_comm_destroy(comm);
}
pub fn allreduce(self: *const Self, T: type, comm: Communicator, buf: []T) void {
    cuda.zg_allreduce(comm, buf.ptr, buf.len, dtype(T), self.context.stream);
}
pub fn reduce_scatter(self: *const Self, T: type, comm: Communicator, send: []const T, recv: []T) void {
    cuda.zg_reduce_scatter(comm, send.ptr, recv.ptr, recv.len, dtype(T), self.context.stream);
}
pub fn all_gather(self: *const Self, T: type, comm: Communicator, send: []const T, recv: []T) void {
    cuda.zg_all_gather(comm, send.ptr, recv.ptr, send.len, dtype(T), self.context.stream);
}

// ---------------------------------------------------------------------- memory
pub fn mem_cache_alloc(self: *Self, T: type, n: usize) !DeviceData(T) {
    const blk = cuda.zg_cache_alloc(self.cache, @max(n * @sizeOf(T), 1), self.context.stream);
    const ptr: [*]T = @ptrCast(@alignCast(blk.ptr orelse return Error.DeviceOOM));
    return .{ .raw = ptr[0..n], .ctx = blk.ctx };
}
pub fn mem_cache_free(self: *Self, data: anytype) void {
    cuda.zg_cache_free(self.cache, .{ .ptr = @ptrCast(data.raw.ptr), .ctx = data.ctx }, self.context.stream);
}
pub fn mem_cache_dupe(self: *Self, T: type, src: []const T) !DeviceData(T) {
    const dst = try self.mem_cache_alloc(T, src.len);
    self.mem_copy(T, src, dst.raw);
    return dst;
}
pub fn mem_alloc(self: *Self, T: type, n: usize) ![]T {
    if (n == 0) return &.{};
    const ptr: [*]T = @ptrCast(@alignCast(cuda.mem_alloc(n * @sizeOf(T), self.context.stream) orelse return Error.DeviceOOM));
    return ptr[0..n];
}
/// One bit per element: ceil(n/8) bytes (src/device/cuda_device.zig mem_alloc_byte_mask).
pub fn mem_alloc_byte_mask(self: *Self, n: usize) ![]u8 {
    return self.mem_alloc(u8, (n + 7) / 8);
}
pub fn mem_dupe(self: *Self, T: type, slice: anytype) ![]T {
    const dst = try self.mem_alloc(T, slice.len);
    self.mem_copy(T, slice, dst);
    return dst;
}
pub fn mem_free(self: *Self, slice: anytype) void {
    if (slice.len == 0) return;
    cuda.mem_free(slice.ptr, self.context.stream);
}
pub fn mem_scratch(self: *Self, T: type, n: usize) []T {
    if (n == 0) return &.{};
    const ptr: [*]T = @ptrCast(@alignCast(cuda.zg_cache_scratch(self.cache, n * @sizeOf(T), self.context.stream) orelse @panic("scratch: device out of memory")));
    return ptr[0..n];
}
pub fn mem_fill(self: Self, T: type, slice: []T, value: T) void {
    var v = value;
    cuda.mem_fill(dtype(T), slice.ptr, slice.len, &v, self.context.stream);
}
pub fn mem_copy(self: Self, T: type, src: []const T, dst: []T) void {
    self.mem_transfer(T, src, dst, .DtoD);
}
pub fn mem_sequence(self: Self, T: type, slice: []T, initial: T, step: T) void {
    var a = initial;
    var b = step;
    cuda.mem_sequence(dtype(T), slice.ptr, slice.len, &a, &b, self.context.stream);
}
pub fn mem_random(self: Self, T: type, slice: []T, op: RandType, rand: std.Random) void {
    cuda.mem_random(dtype(T), slice.ptr, slice.len, if (op == .normal) cuda.NORMAL else cuda.UNIFORM, rand.int(u32), self.context.stream);
}
pub fn mem_take(self: Self, T: type, src: []const T, idxs: []const usize, dst: []T) void {
    cuda.mem_take(dtype(T), src.ptr, src.len, idxs.ptr, idxs.len, dst.ptr, self.context.stream);
}
pub fn mem_transfer(self: Self, T: type, src: []const T, dst: []T, direction: TransferDirection) void {
    const n = src.len * @sizeOf(T);
    switch (direction) {
        .HtoD => cuda.memcpy_HtoD(dst.ptr, src.ptr, n, self.context.stream),
        .DtoH => cuda.memcpy_DtoH(dst.ptr, src.ptr, n, self.context.stream),
        .DtoD => cuda.memcpy_DtoD(dst.ptr, src.ptr, n, self.context.stream),
    }
}
pub fn clear_cache(self: *Self) void {
    cuda.zg_cache_clear(self.cache);
}
pub fn sync(self: Self) void {
    cuda.stream_synchronize(self.context.stream);
    self.check();
}
pub fn is_compatible(self: *const Self, other: *const Self) bool {
    return self.context.device_number == other.context.device_number;
}

/// CUDA-graph capture of the device stream (open / save / run / free).
const ExecutionGraph = struct {
    wrapper: ?cuda.GraphWrapper = null,
    saved: bool = false,

    pub fn open(self: *ExecutionGraph, dev: *Self) void {
        self.free(dev);
        dev.sync();
        self.wrapper = cuda.open_capture(dev.context.stream);
        self.saved = false;
    }
    pub fn save(self: *ExecutionGraph, dev: *Self) void {
        if (self.wrapper) |w| if (!self.saved) {
            cuda.save_capture(w, dev.context.stream);
            self.saved = true;
        };
    }
    pub fn run(self: *ExecutionGraph, dev: *Self) error{ CaptureInProgress, UndefinedCapture }!void {
        const w = self.wrapper orelse return error.UndefinedCapture;
        if (!self.saved) return error.CaptureInProgress;
        cuda.run_capture(w, dev.context.stream);
    }
    pub fn free(self: *ExecutionGraph, dev: *Self) void {
        self.save(dev);
        if (self.wrapper) |w| {
            dev.sync();
            cuda.free_capture(w, dev.context.stream);
            self.wrapper = null;
        }
    }
};
