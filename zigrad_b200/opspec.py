"""Operation parameter structs of the device interface.

Python mirror of ``src/device/opspec.zig``: one class per op, the same field
names, and the ``__name__`` that ``DeviceReference.dispatch`` uses to select
the device method (``src/device/device_reference.zig:15-27``).  Slice fields
hold :class:`zigrad_b200.device.DeviceSlice` objects (pointer + length +
dtype) instead of Zig slices.

The last section holds the ops this backend ADDS to the interface (the
reference runs them as host loops): ``softmax_ce``, ``smooth_l1``, ``sgd``,
``adam``, ``linear``, ``mlp_tail``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional, Sequence


def _op(name):
    def wrap(cls):
        cls = dataclass(cls)
        cls.__name__ = name
        cls.op_name = name
        return cls
    return wrap


# ---- binary element-wise (opspec.zig:19-57)
@_op("add")
class add:
    x: Any
    y: Any
    z: Any


@_op("sub")
class sub:
    x: Any
    y: Any
    z: Any


@_op("mul")
class mul:
    x: Any
    y: Any
    z: Any


@_op("div")
class div:
    x: Any
    y: Any
    z: Any


# ---- linear algebra (opspec.zig:66-203)
@_op("dot")
class dot:
    x: Any
    y: Any
    z: Any


@_op("axpy")
class axpy:
    x: Any
    y: Any
    alpha: float  # the Zig struct holds *const T; a Python float or a DeviceSlice (device scalar)


@_op("outer")
class outer:
    x: Any
    y: Any
    A: Any
    alpha: float


@_op("transpose")
class transpose:
    A: Any
    B: Any
    m: int
    n: int
    alpha: float


@_op("matvec")
class matvec:
    A: Any
    x: Any
    y: Any
    m: int
    n: int
    trans_a: bool
    alpha: float
    beta: float


@_op("matmul")
class matmul:
    A: Any
    B: Any
    C: Any
    m: int
    n: int
    k: int
    trans_a: bool
    trans_b: bool
    lda: int
    ldb: int
    ldc: int
    alpha: float
    beta: float


@_op("bmm_acc")
class bmm_acc:
    A: Any
    B: Any
    C: Any
    A_shape: Sequence[int]
    B_shape: Sequence[int]
    C_shape: Sequence[int]
    trans_a: bool
    trans_b: bool
    lda: int
    ldb: int
    ldc: int
    alpha: float
    beta: float


@_op("sum")
class sum:  # noqa: A001  (name fixed by the interface)
    x: Any
    y: Any


@_op("scale")
class scale:
    x: Any
    alpha: float


@_op("nrm2")
class nrm2:
    x: Any
    y: Any


@_op("clip_nrm2")
class clip_nrm2:
    x: Any
    max_norm: float
    delta: float


# ---- non-linear (opspec.zig:205-475)
@_op("pow_fwd")
class pow_fwd:
    x: Any
    exp: float
    y: Any


@_op("pow_fwd_")
class pow_fwd_:
    x: Any
    exp: float


@_op("pow_bwd")
class pow_bwd:
    x: Any
    x_g: Any
    exp: float
    y_g: Any
    eps: float


@_op("sqrt_fwd_")
class sqrt_fwd_:
    x: Any


@_op("sqrt_fwd")
class sqrt_fwd:
    x: Any
    y: Any


@_op("sqrt_bwd")
class sqrt_bwd:
    x: Any
    x_g: Any
    y_g: Any
    eps: float


@_op("rsqrt_fwd")
class rsqrt_fwd:
    x: Any
    y: Any
    eps: float


@_op("rsqrt_bwd")
class rsqrt_bwd:
    x: Any
    x_g: Any
    y_g: Any
    eps: float


@_op("exp_fwd")
class exp_fwd:
    x: Any
    y: Any


@_op("exp_bwd")
class exp_bwd:
    x_g: Any
    y: Any
    y_g: Any


@_op("relu_fwd")
class relu_fwd:
    x: Any
    y: Any


@_op("relu_bwd")
class relu_bwd:
    x: Any
    x_g: Any
    y_g: Any


@_op("relu_inplace_bwd")
class relu_inplace_bwd:
    x: Any
    x_g: Any


@_op("tanh_fwd")
class tanh_fwd:
    x: Any
    y: Any


@_op("tanh_bwd")
class tanh_bwd:
    x_g: Any
    y: Any
    y_g: Any


@_op("tanh_inplace_bwd")
class tanh_inplace_bwd:
    x: Any
    x_g: Any


@_op("sigm_inplace_bwd")
class sigm_inplace_bwd:
    x: Any
    x_g: Any


@_op("sigm_fwd")
class sigm_fwd:
    x: Any
    y: Any


@_op("sigm_bwd")
class sigm_bwd:
    x_g: Any
    y: Any
    y_g: Any


@_op("max_fwd")
class max_fwd:
    x: Any
    y: Any


@_op("max_bwd")
class max_bwd:
    x: Any
    x_g: Any
    y: Any
    y_g: Any


@_op("clamp_fwd")
class clamp_fwd:
    x: Any
    y: Any
    min: float
    max: float


@_op("clamp_bwd")
class clamp_bwd:
    x: Any
    x_g: Any
    y_g: Any
    min: float
    max: float


@_op("clamp_mask_fwd")
class clamp_mask_fwd:
    x: Any
    y: Any
    min: float
    max: float
    mask: Any  # u8 device slice of ceil(n/8) bytes (mem_alloc_byte_mask)


@_op("clamp_mask_bwd")
class clamp_mask_bwd:
    x_g: Any
    y_g: Any
    mask: Any


@_op("relu_mask_fwd")
class relu_mask_fwd:
    x: Any
    mask: Any


@_op("relu_mask_bwd")
class relu_mask_bwd:
    x_g: Any
    mask: Any


# ---- shape-aware reductions (opspec.zig:477-531)
@_op("unbroadcast")
class unbroadcast:
    x: Any
    x_shape: Sequence[int]
    y: Any
    y_shape: Sequence[int]
    scratch: Any
    alpha: float = 1.0
    beta: float = 0.0


@_op("broadcast")
class broadcast:
    x: Any
    x_shape: Sequence[int]
    y: Any
    y_shape: Sequence[int]
    alpha: float = 1.0
    beta: float = 0.0


@_op("sum_along")
class sum_along:
    x: Any
    x_shape: Sequence[int]
    y: Any
    y_shape: Sequence[int]
    dim: int
    alpha: float = 1.0
    beta: float = 0.0


@_op("max_along")
class max_along:
    x: Any
    x_shape: Sequence[int]
    y: Any
    y_shape: Sequence[int]
    dim: int
    alpha: float = 1.0
    beta: float = 0.0


# ---- index ops (opspec.zig:533-659)
@_op("scatter_add")
class scatter_add:
    src: Any
    offsets: Any
    dst: Any


@_op("scatter_add_2d")
class scatter_add_2d:
    src: Any       # [n_blocks, stride]
    indices: Any   # u64 [n_blocks]
    dst: Any       # [n_segments, stride]
    stride: int


@_op("scatter_add_csr")
class scatter_add_csr:
    src: Any       # [n_segments]
    row_ptr: Any   # u64 [n_segments + 1]
    dst: Any       # [total_elements]


@_op("segment_sum_csr")
class segment_sum_csr:
    src: Any          # [total_elems]
    row_offsets: Any  # u64 [n_segments + 1]
    dst: Any          # [n_segments]


@_op("scatter_gcn_deg_scaled")
class scatter_gcn_deg_scaled:
    dst: Any
    h: Any
    deg: Any
    src_indices: Any
    tgt_indices: Any
    stride: int
    n_edge: int


@_op("scatter_gcn_deg_scaled_bwd")
class scatter_gcn_deg_scaled_bwd:
    grad_output: Any
    h: Any
    deg: Any
    src_indices: Any
    tgt_indices: Any
    grad_h: Any
    grad_deg: Any
    stride: int
    n_edge: int


# ---------------------------------------------------------------------------
# ops added by this backend (host loops in the reference)
# ---------------------------------------------------------------------------
@_op("softmax_ce")
class softmax_ce:
    """src/nn/loss.zig:130-215 as one device op.  ``labels`` is a one-hot
    fp32 [rows, C] slice or a u64 index slice [rows]; ``loss`` a 1-element
    slice; ``grad`` (optional) receives (p - t)/loss_div."""
    logits: Any
    labels: Any
    rows: int
    classes: int
    loss: Any
    grad: Optional[Any] = None
    loss_div: Optional[float] = None
    accumulate: bool = True
    probs: Optional[Any] = None
    ld: int = 0                      # row stride of logits / grad / probs (0 = classes)
    bias_grad: Optional[Any] = None  # [classes]: column sums of the gradient written


@_op("mlp_tail")
class mlp_tail:
    """The last two Linear layers of an MLP with their loss and the backward pass
    down to the gradient of the layer before them, as one device op
    (zg_mlp_tail_fwd_bwd): act1 = relu(act0 W1^T + b1), logits = act1 W2^T + b2,
    softmax cross-entropy forward/backward, dact1, dact0 and the three bias
    gradients (added into db2 / db1 / db0)."""
    act0: Any       # [rows, h1]
    W1: Any         # [h2, h1]
    b1: Any
    W2: Any         # [classes, h2]
    b2: Any
    labels: Any     # one-hot fp32 [rows, classes] or u64 [rows]
    rows: int
    h1: int
    h2: int
    classes: int
    ld_out: int     # row stride of logits / dlogits
    loss_div: float
    act1: Any
    logits: Any
    loss: Any
    dlogits: Any
    dact1: Any
    dact0: Any
    db2: Any
    db1: Any
    db0: Any
    weights_ready: bool = False


@_op("smooth_l1")
class smooth_l1:
    """src/nn/loss.zig:259-305."""
    pred: Any
    target: Any
    beta: float
    loss: Any
    grad: Optional[Any] = None


@_op("sgd")
class sgd:
    """SGD.update over a flat parameter set (src/nn/optim.zig:100-122)."""
    params: Any
    grads: Any
    segments: Sequence[tuple]
    lr: float
    clip: bool = False
    max_norm: float = 10.0
    delta: float = 1e-6
    norms: Optional[Any] = None
    zero_grads: bool = False  # also clear the applied gradients (the next step's zero_grad)


@_op("adam")
class adam:
    """Adam.update over a flat parameter set (src/nn/optim.zig:177-234)."""
    params: Any
    grads: Any
    m: Any
    v: Any
    segments: Sequence[tuple]
    t_first: int
    lr: float
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    clip: bool = False
    max_norm: float = 10.0
    delta: float = 1e-6
    norms: Optional[Any] = None
    bf16_copy: Optional[Any] = None
    step_counter: Optional[Any] = None  # device u64: tensor updates so far (graph-replay safe step count)
    advance_counter: bool = True  # False: read step_counter without advancing it (one optimizer step as several calls, see zg_adam_step_part)


@_op("csr_gcn_propagate")
class csr_gcn_propagate:
    """scatter_gcn_deg_scaled / its grad_h (src/device/host_device.zig:1356-1403)
    over a CSR form of the static edge list, without atomics.  transpose=False:
    rows = targets (forward); True: rows = sources (gradient w.r.t. h)."""
    out: Any
    x: Any
    deg: Any
    row_ptr: Any
    col_idx: Any
    n_rows: int
    n_feat: int
    ld_x: int
    ld_out: int
    transpose: bool = False
    epilogue: str = "none"   # none | bias | bias_relu
    bias: Optional[Any] = None


@_op("linear")
class linear:
    """bmm_acc with a fused epilogue: the Linear layer's three device calls
    (bmm_acc, add, relu_fwd; examples/mnist/src/model.zig:104-110) or a
    backward GEMM with the ReLU mask applied to its result."""
    A: Any
    B: Any
    C: Any
    m: int
    n: int
    k: int
    trans_a: bool
    trans_b: bool
    lda: int
    ldb: int
    ldc: int
    alpha: float = 1.0
    beta: float = 0.0
    epilogue: str = "none"  # none | bias | bias_relu | relu_mask
    bias: Optional[Any] = None
    mask_src: Optional[Any] = None
    n_batch: tuple = field(default=(1, 1, 1))
    colsum: Optional[Any] = None  # fp32 [n]: column sums of the stored C are added here (a bias gradient)
    sm_budget: int = 0  # > 0: size the split-K grid for this many SMs (GEMMs that run side by side on parallel streams share them)
