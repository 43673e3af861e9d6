"""Python faces of the CUDA kernels: each function checks its tensors, passes
raw pointers and the current stream to the exported C function, and raises on
a non-zero return.  Nothing here computes; there is no other code path.
"""
from __future__ import annotations

import contextlib
import ctypes
import functools
import os
from typing import Optional, Tuple

import torch

from .build import library

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dtype}")


_scope_stream = [None]


def _stream() -> int:
    s = _scope_stream[0]
    return s if s is not None else torch.cuda.current_stream().cuda_stream


@contextlib.contextmanager
def stream_scope():
    """Within the scope every launch goes to the stream that was current on entry: the question is asked
    once for a whole forward pass instead of once per kernel."""
    before = _scope_stream[0]
    _scope_stream[0] = torch.cuda.current_stream().cuda_stream
    try:
        yield
    finally:
        _scope_stream[0] = before


# Argument types of the exported C functions: p pointer, i int, l long long, u unsigned long long, f float;
# the last argument of every function is the stream.  Declared once per library, so that a launch passes
# plain Python integers and floats (a pointer is `tensor.data_ptr()`, None is a null pointer).
_SIGNATURES = {
    "jb_embed_gather": "pippiippfp", "jb_rmsnorm": "pppifpiiiplp", "jb_residual_add": "ppilp",
    "jb_swiglu": "ppiiip", "jb_swiglu_f32_to_bf16": "piipiip", "jb_zero_f32": "plp",
    "jb_pack_weight_bf16": "piipp", "jb_rope_cache_write": "piipipppppiiiiiiip",
    "jb_gemm_f32": "pppiiiiiip", "jb_attention_f32": "pppppppiiiiiiififfp",
    "jb_gemm_bf16": "pplipiiiiiiplpiffpp", "jb_gemm_bf16_pair": "pplipiiiiiiiffpp",
    "jb_gemm_bf16_pair_grouped": "pplipiiiiipiffpp", "jb_expert_plan": "piiiippppp",
    "jb_gemm_bf16_pair_qkv_rope": "ppliippppppiiiipp",
    "jb_sample": "piipfiffppupppp",
    "jb_attention_bf16_prefill": "pppppppiiiiiiiifp", "jb_attention_bf16_decode": "ppppppppiiiiiiifip",
    "jb_attention_bf16_decode_fused": "pipppppppppiiiiiiifiip",
    "jb_attention_bf16_prefill_capped": "pppppppiiiiiiiififfp", "jb_attention_bf16_decode_capped": "ppppppppiiiiiiifiiffp",
    "jb_join_norm": "pppppffpppfipipiiplplp", "jb_head_norm_gate": "ppipipfipiiiip", "jb_sigmoid_gate": "pipiiiiip",
    "jb_head_norm_rope_cache": "pippfpippipppiiiiiiiiifip",
    "jb_delta_rule": "piiiipiiippfppllppiiiiip",
    "jb_route_topk": "piiippiiiip", "jb_experts_few_tokens": "pippipppippiiiiffip", "jb_expert_gather": "pippipiip",
    "jb_expert_scatter": "pppipiip",
    "jb_gla_decay": "piiippfpiip", "jb_exp_gates": "piiippfppllppiip",
    "jb_gated_linear_scan": "piiiifpiippplppiiiiiippp", "jb_scale_rows_sigmoid": "pipiiip",
    "jb_attention_tc_prefill": "pppppppiiiiiiiiiifpp", "jb_attention_tc_prefill_capped": "pppppppiiiiiiiiiififfpp",
    "jb_streams_rmsnorm": "pppipifpiiipplp", "jb_streams_mix": "ppppiiip", "jb_streams_mix_rmsnorm": "pppppipifpiiiplp", "jb_embed_streams": "pippiiippp",
    "jb_lightning_scan": "piiiipppppiiiiiipp", "jb_gated_rmsnorm": "ppipifpiiip",
    "jb_conv_rope_cache": "pipipipppppippppiiiiiiip", "jb_conv_state_update": "pipippiip",
    "jb_diff_attention": "pppipipppiiiiiiiiiffffp",
    "jb_diff_attention_prefill": "pppppppiiiiiiiiiiffffp",
    "jb_clamped_glu": "piipiiiffp",
    "jb_sublayer_norm_add": "ppiffppiiiplplp", "jb_qk_norm_rope_cache": "pippppfpippipppiiiiiiip",
    "jb_latent_prep": "piiiipfpippiip", "jb_causal_conv_silu": "piiippipllppppiiiip",
    "jb_mamba2_scan": "piiipipppppllppiiiiiiippp", "jb_gated_group_rmsnorm": "ppipfpiiiip", "jb_pad_rows_bf16": "pipiip", "jb_scale_softcap": "plffp",
}
_CTYPES = {"p": ctypes.c_void_p, "i": ctypes.c_int, "l": ctypes.c_longlong, "u": ctypes.c_ulonglong,
           "f": ctypes.c_float}

_libs = {}


def _lib(stem: str, key=None, defines=None) -> ctypes.CDLL:
    """The built library `stem` (variant `key`, compiled with `defines(key)` or the dict `defines`);
    asked for on every launch, so the answer is remembered here."""
    lib = _libs.get((stem, key))
    if lib is None:
        lib = library(stem, defines(key) if callable(defines) else defines)
        for name, signature in _SIGNATURES.items():
            fn = getattr(lib, name, None)
            if fn is not None:
                fn.argtypes = [_CTYPES[c] for c in signature]
                fn.restype = ctypes.c_int
        _libs[(stem, key)] = lib
    return lib


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# Whether the faces below check their tensors (device, contiguity, dtype, shape).  The engine turns the
# checks off for a step whose shape it has run before with the checks on: the same parts then hand the same
# kinds of tensors to the same kernels.
_checks = [True]


@contextlib.contextmanager
def unchecked():
    before = _checks[0]
    _checks[0] = False
    try:
        yield
    finally:
        _checks[0] = before


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if not _checks[0]:
        return
    if not t.is_cuda:
        raise KernelError(f"{name}: tensor must be on a CUDA device (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{name}: expected shape {tuple(shape)}, got {tuple(t.shape)}")


_launches = [0]


def launch_count() -> int:
    """Kernels of this library launched (or captured into a graph) so far."""
    return _launches[0]


_trace = [None]    # while a step is profiled: the list that takes (face, kernels, event after the launch)


@contextlib.contextmanager
def trace_launches():
    """Within the scope every launch of this library is followed by a CUDA event on the current stream; the
    list that is handed out holds (face, kernels, event), led by an event recorded on entry.  The time between
    two events is the time the stream spent on the launch between them (kernels run one after another on a
    stream; what overlaps under programmatic dependent launch is counted for the later kernel)."""
    before = _trace[0]
    start = torch.cuda.Event(enable_timing=True)
    start.record()
    events = [("start", 0, start)]
    _trace[0] = events
    try:
        yield events
    finally:
        _trace[0] = before


def _check(code: int, what: str, kernels: int = 1) -> None:
    if code == 0:
        _launches[0] += kernels
        if _trace[0] is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            _trace[0].append((what, kernels, ev))
        return
    if code >= 10000:
        names = {10001: "size not supported (see stderr)", 10002: "dtype not supported",
                 10003: "tensor map could not be encoded"}
        raise KernelError(f"{what}: {names.get(code, 'error')} (code {code})")
    raise KernelError(f"{what}: CUDA error {code}")


# -- embedding, norm, elementwise ---------------------------------------------
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor,
                 feedback: Optional[torch.Tensor] = None, token_slot: Optional[torch.Tensor] = None,
                 scale: float = 1.0) -> None:
    """out[t, :] = float32(table[ids[t], :]) * scale; a negative id stands for feedback[token_slot[t]]"""
    T, H = out.shape
    _need(table, "embed table")
    _need(ids, "token ids", torch.int32, (T,))
    _need(out, "embed out", torch.float32)
    if table.shape[1] != H:
        raise KernelError(f"embed: table width {table.shape[1]} != output width {H}")
    _check(_lib("elementwise").jb_embed_gather(
        _ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out), T, H, _ptr(feedback), _ptr(token_slot),
        float(scale), _stream()), "embed_gather")


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float, out: torch.Tensor,
            row_index: Optional[torch.Tensor] = None, clear: Optional[torch.Tensor] = None) -> None:
    """out[r] = x[row_index[r] or r] / sqrt(mean(x^2) + eps) * gamma.  `clear`: a float32
    scratch tensor (whole 16-byte vectors) that the same launch sets to zero."""
    rows, H = out.shape
    _need(x, "rmsnorm x", torch.float32)
    _need(gamma, "rmsnorm gamma", None, (H,))
    _need(out, "rmsnorm out")
    if x.shape[1] != H:
        raise KernelError(f"rmsnorm: input width {x.shape[1]} != output width {H}")
    if clear is not None:
        _need(clear, "rmsnorm clear", torch.float32)
    if row_index is not None:
        _need(row_index, "rmsnorm row_index", torch.int32, (rows,))
    elif x.shape[0] < rows:
        raise KernelError("rmsnorm: fewer input rows than output rows")
    _check(_lib("elementwise").jb_rmsnorm(
        _ptr(x), _ptr(row_index), _ptr(gamma), dtype_code(gamma.dtype), eps, _ptr(out),
        dtype_code(out.dtype), rows, H, _ptr(clear), 0 if clear is None else clear.numel(),
        _stream()), "rmsnorm")


def residual_add(residual: torch.Tensor, delta: torch.Tensor) -> None:
    """residual += float32(delta), elementwise, in place"""
    _need(residual, "residual", torch.float32)
    _need(delta, "delta", None, residual.shape)
    _check(_lib("elementwise").jb_residual_add(
        _ptr(residual), _ptr(delta), dtype_code(delta.dtype), residual.numel(), _stream()),
        "residual_add")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, c] = silu(gate_up[t, c]) * gate_up[t, I + c]"""
    T, I = out.shape
    _need(gate_up, "swiglu input", out.dtype, (T, 2 * I))
    _need(out, "swiglu out")
    _check(_lib("elementwise").jb_swiglu(_ptr(gate_up), _ptr(out), dtype_code(out.dtype), T, I, _stream()),
           "swiglu")


def swiglu_f32_to_bf16(gate_up: torch.Tensor, out: torch.Tensor, up_col: int) -> None:
    """out[t, c] = silu(gate_up[t, c]) * gate_up[t, up_col + c]; float32 in, bfloat16 out."""
    T, I = out.shape
    _need(gate_up, "swiglu input", torch.float32)
    _need(out, "swiglu out", torch.bfloat16)
    if gate_up.dim() != 2 or gate_up.shape[0] != T:
        raise KernelError(f"swiglu: input of shape {tuple(gate_up.shape)} does not hold {T} rows")
    _check(_lib("elementwise").jb_swiglu_f32_to_bf16(_ptr(gate_up), gate_up.shape[1], int(up_col), _ptr(out), T, I,
                                                      _stream()), "swiglu_f32_to_bf16")


def zero_f32(t: torch.Tensor) -> None:
    """Fill a float32 tensor with zeros (whole 16-byte vectors)."""
    _need(t, "zero target", torch.float32)
    _check(_lib("elementwise").jb_zero_f32(_ptr(t), t.numel(), _stream()), "zero_f32")


# -- rotary positions + cache append --------------------------------------------
def rope_cache_write(qkv: torch.Tensor, q_out: torch.Tensor, cos_sin: Optional[torch.Tensor],
                     positions: torch.Tensor, dest: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                     v_cache: Optional[torch.Tensor], nh: int, nkv: int, hd: int, page_size: int,
                     write_kv: bool = True) -> None:
    T = q_out.shape[0]
    width = (nh + 2 * nkv) * hd if write_kv else nh * hd
    _need(qkv, "qkv")
    if qkv.shape[0] != T or qkv.shape[1] < width:
        raise KernelError(f"rope: qkv shape {tuple(qkv.shape)} does not hold {T} rows of width {width}")
    _need(q_out, "q_out", None, (T, nh * hd))
    _need(positions, "positions", torch.int32, (T,))
    rotate = cos_sin is not None
    if rotate:
        _need(cos_sin, "rope table", torch.float32)
        if cos_sin.shape[1:] != (hd // 2, 2):
            raise KernelError(f"rope: table shape {tuple(cos_sin.shape)} does not fit head_dim {hd}")
    if write_kv:
        _need(dest, "cache rows", torch.int32, (T,))
        _need(k_cache, "k cache", q_out.dtype)
        _need(v_cache, "v cache", q_out.dtype)
    _check(_lib("rope_cache").jb_rope_cache_write(
        _ptr(qkv), qkv.shape[1], dtype_code(qkv.dtype), _ptr(q_out), dtype_code(q_out.dtype), _ptr(cos_sin),
        _ptr(positions), _ptr(dest), _ptr(k_cache), _ptr(v_cache),
        T, nh, nkv, hd, page_size, int(rotate), int(write_kv), _stream()), "rope_cache_write")


# -- float32 matrix product and attention ------------------------------------------
def gemm_f32(x: torch.Tensor, w: torch.Tensor, y: torch.Tensor, accumulate: bool = False, label: str = "") -> None:
    """y[T, N] (+)= x[T, K] . w[N, K]^T in true float32 (`label`: what a profile of a step calls this product)"""
    T, K = x.shape
    N = w.shape[0]
    _need(x, "gemm x", torch.float32)
    _need(w, "gemm w", torch.float32, (N, K))
    _need(y, "gemm y", torch.float32, (T, N))
    _check(_lib("gemm_f32").jb_gemm_f32(_ptr(x), _ptr(w), _ptr(y), T, N, K, K, N, int(accumulate), _stream()),
           "gemm_f32 " + label if label else "gemm_f32")


def attention_f32(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                  block_table: torch.Tensor, token_slot: torch.Tensor, positions: torch.Tensor,
                  nh: int, nkv: int, hd: int, page_size: int, window: int, scale: float, chunk: int = 0,
                  softcap: float = 0.0, sink: bool = False) -> None:
    """`chunk` > 0: a query sees only the keys of its own chunk of positions, [floor(pos / chunk) chunk, pos];
    `softcap` > 0: a score s becomes softcap tanh(s / softcap); `sink`: the softmax's denominator has one more
    term, exp(0), a key of score 0 that has no value."""
    T = q.shape[0]
    _need(q, "attention q", torch.float32, (T, nh * hd))
    _need(out, "attention out", torch.float32, (T, nh * hd))
    _need(k_cache, "k cache", torch.float32)
    _need(v_cache, "v cache", torch.float32)
    _need(block_table, "block table", torch.int32)
    _need(token_slot, "token slots", torch.int32, (T,))
    _need(positions, "positions", torch.int32, (T,))
    _check(_lib("attention_f32").jb_attention_f32(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _ptr(token_slot), _ptr(positions),
        T, nh, nkv, hd, page_size, block_table.shape[1], int(window), scale, int(chunk), float(softcap),
        1.0 if sink else 0.0, _stream()), "attention_f32")


# -- bfloat16 tensor-core matrix product --------------------------------------------
_status = {}
SM_COUNT_TARGET = 296      # CTAs wanted in flight for a weight-streaming product (two per SM)


_bound_device = []


def bind_device(device: torch.device) -> None:
    """One process drives one GPU: the kernel libraries set their kernels up (shared-memory limits, occupancy,
    SM count) for the device of their first launch and keep that.  The first model names the device; a model
    on another device is refused here, not at some launch."""
    index = torch.device(device).index
    index = torch.cuda.current_device() if index is None else index
    if not _bound_device:
        _bound_device.append(index)
    elif _bound_device[0] != index:
        raise KernelError(f"this process already runs its kernels on cuda:{_bound_device[0]}; a model on "
                          f"cuda:{index} needs a process of its own (the library drives one GPU per process)")


def kernel_status(device: torch.device) -> torch.Tensor:
    """Device int that a kernel sets when one of its bounded waits ran out."""
    st = _status.get(device)
    if st is None:
        st = torch.zeros(1, dtype=torch.int32, device=device)
        _status[device] = _status[st.device] = st       # "cuda" and "cuda:0" name the same word
    return st


def check_kernel_status(device: torch.device) -> None:
    """Synchronises; raises if a tensor-core kernel gave up on a wait."""
    code = int(kernel_status(device).item())
    if code != 0:
        kernel_status(device).zero_()
        who = {1: "TMA producer", 2: "MMA issuer", 3: "epilogue"}.get(code % 10, "?")
        raise KernelError(f"a tensor-core kernel timed out waiting on an mbarrier ({who}, code {code})")


class PackedWeight:
    """A [rows, cols] bfloat16 matrix laid out for the tensor-core products: tiles of 128 rows x 64 columns,
    each one contiguous, zero-padded and already swizzled 16 KB block, stored [row tile][k tile]
    (`pack_weight`).  A stage of a product then reads its weights as one sequential block of HBM.
    `up_tile_offset` > 0 marks a gated pair: the gate matrix's row tiles first, the up matrix's row tiles
    from there on (`rows` counts one of the two)."""

    def __init__(self, tiles: torch.Tensor, rows: int, cols: int, up_tile_offset: int = 0):
        self.tiles, self.rows, self.cols, self.up_tile_offset = tiles, int(rows), int(cols), int(up_tile_offset)

    @property
    def n_tiles(self) -> int:
        return self.tiles.shape[0] * self.tiles.shape[1]

    @property
    def device(self):
        return self.tiles.device

    def nbytes(self) -> int:
        return self.tiles.numel() * 2

    def first_rows(self, rows: int) -> "PackedWeight":
        """The matrix of the first `rows` rows (shares storage; a last tile may hold further rows, which
        the product's epilogue leaves out)."""
        if rows > self.rows or self.up_tile_offset:
            raise KernelError(f"first_rows({rows}) of a packed matrix of {self.rows} rows")
        return PackedWeight(self.tiles[: (rows + 127) // 128], rows, self.cols)

    def stacked(self) -> "PackedWeight":
        """A gated pair as the plain matrix of its row tiles: the gate rows (padded to whole tiles of 128),
        then the up rows from row 128 * up_tile_offset on (shares storage)."""
        if not self.up_tile_offset:
            raise KernelError("stacked(): the weight is no gated pair")
        return PackedWeight(self.tiles, self.tiles.shape[0] * 128, self.cols)


def pack_weight(w: torch.Tensor) -> PackedWeight:
    """Row-major bfloat16 [N, K] (K a multiple of 8) -> PackedWeight."""
    _need(w, "weight to pack", torch.bfloat16)
    if w.dim() != 2 or w.shape[1] % 8:
        raise KernelError(f"pack_weight: a matrix whose width is a multiple of 8 is needed, got {tuple(w.shape)}")
    N, K = w.shape
    tiles = torch.empty(((N + 127) // 128, (K + 63) // 64, 128, 64), dtype=torch.bfloat16, device=w.device)
    _check(_lib("elementwise").jb_pack_weight_bf16(_ptr(w), N, K, _ptr(tiles), _stream()), "pack_weight")
    return PackedWeight(tiles, N, K)


def pack_gated(gate: torch.Tensor, up: torch.Tensor) -> PackedWeight:
    """Gate and up matrices of equal shape as one PackedWeight (gate tiles, then up tiles)."""
    if gate.shape != up.shape:
        raise KernelError(f"pack_gated: shapes {tuple(gate.shape)} and {tuple(up.shape)} differ")
    g, u = pack_weight(gate), pack_weight(up)
    return PackedWeight(torch.cat([g.tiles, u.tiles], dim=0), gate.shape[0], gate.shape[1], g.tiles.shape[0])


# JANUS_DETERMINISTIC=1 (or `set_deterministic(True)` before a model is built): the slices of a cut K are
# summed in the fixed order of the slices instead of by atomic adds in the order they happen to finish, so the
# same requests give the same bits.  Every slice leaves its tile in scratch; the one that arrives last at the
# output tile's ticket adds them up (single-CTA kernel; CTA pairs then run uncut).
_deterministic = [os.environ.get("JANUS_DETERMINISTIC", "0") == "1"]


def set_deterministic(flag: bool) -> None:
    """Switch cutting of K (atomic adds) off or on for products launched from now on; decode steps that an
    engine has already captured into CUDA graphs keep what they were captured with."""
    _deterministic[0] = bool(flag)
    gemm_plan.cache_clear()


def is_deterministic() -> bool:
    return _deterministic[0]


ORDERED_SCRATCH_MAX_BYTES = 256 << 20
_ORDERED_TICKETS = 1 << 16
_ordered_scratch = {}     # device -> (partials, tickets); outgrown buffers stay alive for captured graphs
_ordered_retired = []


def _ordered_buffers(device: torch.device, floats: int):
    """Scratch for ordered sums of `floats` floats on `device` (None if that is more than the cap)."""
    if floats * 4 > ORDERED_SCRATCH_MAX_BYTES:
        return None
    have = _ordered_scratch.get(device)
    if have is None or have[0].numel() < floats:
        size = max(floats, 2 * have[0].numel() if have is not None else (8 << 20) // 4)
        size = min(size, ORDERED_SCRATCH_MAX_BYTES // 4)
        tickets = have[1] if have is not None else torch.zeros(_ORDERED_TICKETS, dtype=torch.int32, device=device)
        if have is not None:
            _ordered_retired.append(have[0])
        have = (torch.empty(size, dtype=torch.float32, device=device), tickets)
        _ordered_scratch[device] = have
    return have


def gated_runs_unfused(T: int, I: int) -> bool:
    """Whether a SiLU-gated product of I features runs as a plain product of the stacked gate and up rows
    into float32 and an activation kernel: decode-sized steps of narrow layers, where the fused kernel's
    tiles (128 features, gate and up rows together) fill less than half of the SMs.  Measured at 8192
    features (64 tiles): 13.6 us against 15.1 at 8 tokens, 17.6 against 21.5 at 64; at 13824 and 14336
    features the fused kernel is faster (45.5 against 45.8 to 51.9, 37.1 against 40.0 to 44.6)."""
    return _GATED_UNFUSED and T <= 64 and 2 * ((I + 127) // 128) <= SM_COUNT_TARGET // 2


_GATED_UNFUSED = os.environ.get("JANUS_GATED_UNFUSED", "1") != "0"


def split_k_for(T: int, N: int, K: int) -> int:
    """How many slices of K an adding product (mode "add", or a float32 "store" run as clear + add) is cut
    into; 1 when it is not cut."""
    return gemm_plan(T, N, K, "add")[1]


# token counts from which the CTA-pair kernel (cta_group::2, 256-row weight tiles) may run a product;
# JANUS_GEMM_PAIR=0 keeps every product on the single-CTA kernel
GEMM_PAIR_MIN_TOKENS = int(os.environ.get("JANUS_GEMM_PAIR_MIN_TOKENS", "65"))
_GEMM_PAIR = os.environ.get("JANUS_GEMM_PAIR", "1") != "0"
# token counts from which the q/k/v projection with rotation and cache append in its epilogue runs
QKV_FUSED_MIN_TOKENS = int(os.environ.get("JANUS_QKV_FUSED_MIN_TOKENS", "512"))

# Constants of the cost estimate in `gemm_plan`.  They were fitted so that the estimate picks the fastest
# of the alternatives (the single-CTA kernel with K in 1, 2, 3, 4, 6 or 8 slices; CTA pairs with K in 1, 2,
# 3, 4 or 6) as measured on a B200 for the four products of 1B-, 8B-, 13B- and 70B-sized layers at 72 to
# 4096 tokens: the pick is 0.4 % slower than the best alternative on average.  They rank alternatives; they
# are no forecast of a time.
_PLAN_SM_FLOPS_PER_US = 6.09e6      # tensor-core rate of one SM on single-CTA tiles, flop per microsecond
_PLAN_SM_FILL_BYTES_PER_US = 1.99e5  # operand bytes one SM takes in per microsecond
_PLAN_TILE_US = 0.0                 # per tile of the single-CTA kernel
_PLAN_PAIR_STEP_US = 0.461          # one 256 x 256 x 64 step of a CTA pair
_PLAN_PAIR_TILE_US = 4.18           # per tile of a CTA pair: first loads, epilogue
_PLAN_HBM_BYTES_PER_US = 6.68e6     # the weight stream
_PLAN_US_PER_ADD = 5.14e-7          # one float32 add of a slice of K into the output, single-CTA kernel
_PLAN_PAIR_US_PER_ADD = 4.26e-7     # the same, CTA pairs
_PLAN_SPLITS = (1, 2, 3, 4, 6, 8)
_PLAN_DECODE_MAX_SPLIT = 24
_PLAN_DECODE_STEPS_PER_ADD = 1e-4   # adds of a 128-row tile's token, in steps along K (fitted: 60 measured cases)
_PLAN_PAIR_SPLITS = (1, 2, 3, 4, 6)
_PLAN_ORDERED_TILE_US = 3.0         # deterministic mode: fence, ticket and ordered sum of a tile of a cut K
_PLAN_TAIL_MIN_K = 32               # k-tiles a slice of a last wave's tile has at least (measured: the o projection
                                    # of 8B layers, 64 k-tiles, loses 4 % with slices of 16; the down projection, 224, gains 12 %)


def gemm_plan(T: int, N: int, K: int, mode: str, allow_pairs: bool = True) -> Tuple[bool, int]:
    """(CTA pairs?, slices of K): see `gemm_plan_whole`, which also says how many tiles stay uncut."""
    return gemm_plan_whole(T, N, K, mode, allow_pairs)[:2]


def _plan_cache_clear() -> None:
    gemm_plan_whole.cache_clear()


gemm_plan.cache_clear = _plan_cache_clear


@functools.lru_cache(maxsize=4096)
def gemm_plan_whole(T: int, N: int, K: int, mode: str, allow_pairs: bool = True) -> Tuple[bool, int, int]:
    """Which kernel runs x[T, K] . w[N, K]^T and into how many slices of K it is cut: (CTA pairs?, slices).

    Up to 64 tokens the product streams its weights: the single-CTA kernel, with K cut so that the waves of
    tiles over the SMs x the steps of a slice are fewest (only a product that adds can be cut; its slices
    meet by atomic adds): 4096 x 4096 makes 32 tiles, and 13 slices of 5 steps in 3 waves beat 9 of 8 in 2.
    Above, the choice is by an estimate of the time: waves of tiles over the SMs x (steps along K x the
    time of a step, tensor-core bound or bound by what an SM takes in per step, + a tile's fixed cost), not
    below the time of the weight stream, plus the atomic adds of a cut K.  Few output tiles (a 4096 x 4096
    matrix and 256 tokens make 32) leave most SMs idle unless K is cut; CTA pairs halve the operand bytes
    per flop and win once their 256 x 256 tiles fill the SMs."""
    tiles_w = (N + 127) // 128
    k_tiles = (K + 63) // 64
    sms = SM_COUNT_TARGET // 2
    ordered = _deterministic[0]     # slices are summed in a fixed order: the single-CTA kernel can, CTA pairs cannot
    if T <= 64:
        if mode != "add" or tiles_w >= sms:
            return False, 1, 0   # a wave of tiles or more streams weights on every SM as it is
        # the critical path in steps along K: waves of tiles over the SMs x steps of a slice; a little per add
        best = (float("inf"), 1)
        for split in range(1, max(1, min(k_tiles // 4, _PLAN_DECODE_MAX_SPLIT)) + 1):
            waves = (tiles_w * split + sms - 1) // sms
            if ordered and split > 1 and waves > 1:
                break     # an ordered sum costs a tile a fence and a ticket (about 3 us): one tile per SM at most
            cost = waves * ((k_tiles + split - 1) // split) + _PLAN_DECODE_STEPS_PER_ADD * split * T * tiles_w
            if cost < best[0] - 1e-9:
                best = (cost, split)
        return False, best[1], 0
    gated = mode == "swiglu"
    w_rows = 2 * N if gated else N
    stream = w_rows * K * 2 / _PLAN_HBM_BYTES_PER_US
    # token tile of the single-CTA kernel (a gated product's two accumulators leave room for 256 tokens in one
    # buffer only, which serves where a CTA has one tile: up to 256 tokens)
    bn = 128 if (T <= 128 or (gated and T > 256)) else 256
    stage_rows = 256 if gated else 128                      # weight rows a step brings in
    step = max(2.0 * stage_rows * bn * 64 / _PLAN_SM_FLOPS_PER_US,
               (stage_rows + bn) * 64 * 2 / _PLAN_SM_FILL_BYTES_PER_US)
    best = (float("inf"), False, 1, 0)
    for split in (_PLAN_SPLITS if mode == "add" else (1,)):
        if split > 1 and split > k_tiles // 4:
            break
        tiles = tiles_w * ((T + bn - 1) // bn) * split
        waves = (tiles + sms - 1) // sms
        cost = max(waves * (((k_tiles + split - 1) // split) * step + _PLAN_TILE_US), stream)
        if split > 1:
            cost += _PLAN_US_PER_ADD * T * N * split + (_PLAN_ORDERED_TILE_US * waves if ordered else 0.0)
        best = min(best, (cost, False, split, 0))
    if allow_pairs and _GEMM_PAIR and T >= GEMM_PAIR_MIN_TOKENS:
        clusters = ((T + 255) // 256) * (tiles_w if gated else (N + 255) // 256)
        for split in (_PLAN_PAIR_SPLITS if mode == "add" and not ordered else (1,)):
            if split > 1 and split > k_tiles // 4:
                break
            waves = (clusters * split + sms // 2 - 1) // (sms // 2)
            cost = max(waves * (((k_tiles + split - 1) // split) * _PLAN_PAIR_STEP_US + _PLAN_PAIR_TILE_US), stream)
            if split > 1:
                cost += _PLAN_PAIR_US_PER_ADD * T * N * split
            best = min(best, (cost, True, split, 0))
        pairs = sms // 2
        whole, tail = clusters // pairs * pairs, clusters % pairs
        if mode == "add" and not ordered and whole and tail:
            # more than a wave of tiles and a last wave that is not full: only that wave's tiles are cut, into
            # slices of at least _PLAN_TAIL_MIN_K k-tiles (shorter pieces are all epilogue)
            for split in _PLAN_PAIR_SPLITS[1:] + (8,):
                per = (k_tiles + split - 1) // split
                if per < _PLAN_TAIL_MIN_K:
                    break
                rounds = (tail * split + pairs - 1) // pairs
                cost = max(whole // pairs * (k_tiles * _PLAN_PAIR_STEP_US + _PLAN_PAIR_TILE_US)
                           + rounds * (per * _PLAN_PAIR_STEP_US + _PLAN_PAIR_TILE_US), stream)
                cost += _PLAN_PAIR_US_PER_ADD * T * N * split * tail / clusters
                best = min(best, (cost, True, split, whole))
    return best[1], best[2], best[3]


def _defines_from_env(name: str) -> dict:
    """Build-time overrides of a kernel's tuning macros for experiments, read once when this module loads,
    e.g. JANUS_GEMM_DEFINES="JB_RING_KB=104,JB_MAX_STAGES=6"; none by default."""
    text = os.environ.get(name, "")
    return {k.strip(): int(v) for k, v in (item.split("=") for item in text.split(",") if item.strip())}


def _defines_key(defines: Optional[dict]):
    return tuple(sorted(defines.items())) if defines else None


_GEMM_DEFINES = _defines_from_env("JANUS_GEMM_DEFINES") or None
_PAIR_DEFINES = _defines_from_env("JANUS_GEMM_PAIR_DEFINES") or None
_ATTN_TC_DEFINES = _defines_from_env("JANUS_ATTN_TC_DEFINES")
_ATTN_DEFINES = _defines_from_env("JANUS_ATTN_DEFINES")
_ATTN_TC = os.environ.get("JANUS_ATTN_TC", "1") != "0"     # 0: prompts attend on the mma.sync kernel


def gemm_bf16(x: torch.Tensor, w: PackedWeight, y: torch.Tensor, mode: str = "store",
              split_k: Optional[int] = None, pair: Optional[bool] = None, whole_tiles: int = 0,
              label: str = "", gate_limit: float = 0.0, gate_alpha: float = 1.0) -> None:
    """bf16 x[T, K] . w[N, K]^T on tcgen05 with float32 accumulation; w packed (`pack_weight`).
    mode "store": y[T, N] = result (bf16 or float32 by y's dtype);
    mode "add":   y[T, N] += result, y float32 (K may be split, sums meet by atomic adds);
    mode "swiglu": w a gated pair (`pack_gated`), y[T, N] = silu(gate) * up in bf16; with gate_limit > 0 the
                   clamped form g sigmoid(gate_alpha g) (u + 1), g = min(gate, limit), u = clamp(up, +-limit).
    `split_k`, `pair`, `whole_tiles`: as `gemm_plan_whole` picks them unless given (`whole_tiles`: CTA pairs
    only, the first so many 256 x 256 output tiles of an adding product stay uncut)."""
    T, K = x.shape
    _need(x, "gemm x", torch.bfloat16)
    _need(y, "gemm y")
    if not isinstance(w, PackedWeight):
        raise KernelError("gemm: the weight must be packed (ops.pack_weight / ops.pack_gated)")
    if w.cols != K:
        raise KernelError(f"gemm: weight of {w.rows} x {w.cols} does not fit K = {K}")
    N = w.rows
    if mode == "swiglu":
        code, want = 3, torch.bfloat16
        if not w.up_tile_offset:
            raise KernelError("gemm swiglu: the weight is no gated pair (ops.pack_gated)")
    else:
        if w.up_tile_offset:
            raise KernelError(f"gemm {mode}: the weight is a gated pair")
        if mode == "add":
            code, want = 2, torch.float32
        elif mode == "store":
            code, want = (1, torch.float32) if y.dtype == torch.float32 else (0, torch.bfloat16)
        else:
            raise KernelError(f"gemm: unknown mode {mode!r}")
    if y.dtype != want or tuple(y.shape) != (T, N):
        raise KernelError(f"gemm {mode}: output must be {want} [{T}, {N}], got {y.dtype} {tuple(y.shape)}")
    if split_k is None:
        if pair is not True:
            pair, split_k, whole_tiles = gemm_plan_whole(T, N, K, mode, allow_pairs=pair is not False)
        else:
            split_k = 1
        if code != 2:
            split_k = 1          # a storing product cut along K is the caller's clear + "add"
    elif pair is None:
        pair = False
    if pair:
        _check(_lib("gemm_bf16_tc2", _defines_key(_PAIR_DEFINES), _PAIR_DEFINES).jb_gemm_bf16_pair(
            _ptr(x), _ptr(w.tiles), w.n_tiles, w.up_tile_offset, _ptr(y), T, N, K, N, code,
            int(split_k), int(whole_tiles), gate_limit, gate_alpha, _ptr(kernel_status(x.device)), _stream()),
            "gemm_bf16_pair " + label if label else "gemm_bf16_pair")
        return
    partials = tickets = None
    if split_k > 1 and _deterministic[0]:
        bn = 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128 if T <= 128 else 256
        k_tiles = (K + 63) // 64
        per = (k_tiles + split_k - 1) // split_k
        slices = (k_tiles + per - 1) // per
        out_tiles = ((N + 127) // 128) * ((T + bn - 1) // bn)
        scratch = _ordered_buffers(x.device, out_tiles * slices * bn * 128) if out_tiles <= _ORDERED_TICKETS else None
        if scratch is None:
            split_k = 1          # too much scratch: K whole
        else:
            partials, tickets = scratch
    _check(_lib("gemm_bf16_tc", _defines_key(_GEMM_DEFINES), _GEMM_DEFINES).jb_gemm_bf16(
        _ptr(x), _ptr(w.tiles), w.n_tiles, w.up_tile_offset, _ptr(y), T, N, K, N, code,
        int(split_k), _ptr(partials), 0 if partials is None else partials.numel(), _ptr(tickets),
        0 if tickets is None else tickets.numel(), gate_limit, gate_alpha, _ptr(kernel_status(x.device)), _stream()),
        "gemm_bf16 " + label if label else "gemm_bf16")


def grouped_max_items(rows: int, groups: int, features: int, mode: str) -> int:
    """A bound on the tiles of a grouped product over `rows` rows in `groups` groups: every group's last tile of 256
    rows may be partly empty."""
    per = (features + 127) // 128 if mode == "swiglu" else (features + 255) // 256
    return (rows // 256 + min(groups, rows)) * per


def gemm_bf16_grouped(x: torch.Tensor, w: PackedWeight, y: torch.Tensor, table: torch.Tensor, max_items: int,
                      mode: str = "store", label: str = "", gate_limit: float = 0.0, gate_alpha: float = 1.0) -> None:
    """A product per group of rows, all in one launch of the CTA-pair kernel: the rows of x [T, K] are sorted into
    groups and w is the packed stack of the groups' matrices ([groups * N, K]; mode "swiglu": a gated pair of two
    such stacks), N a multiple of 128.  `table` (int32 on the device, made by a kernel earlier in the stream, e.g.
    `expert_plan`) holds its count of items in [0] and item i as (first row, end of the group's rows, first weight
    row in the stack, first column of y) at [4 + 4 i]; `max_items` bounds the count (`grouped_max_items`).
    y [T, N]: bfloat16 (mode "swiglu", or "store") or float32 ("store")."""
    T, K = x.shape
    _need(x, "grouped gemm x", torch.bfloat16)
    _need(y, "grouped gemm y")
    _need(table, "grouped gemm table", torch.int32)
    if not isinstance(w, PackedWeight) or w.cols != K:
        raise KernelError("grouped gemm: the weight must be packed and as wide as x")
    N = y.shape[1]
    if y.shape[0] != T or N % 128 or w.rows % N or table.numel() < 4 + 4 * max_items:
        raise KernelError(f"grouped gemm: y {tuple(y.shape)}, a stack of {w.rows} rows, a table of {table.numel()} ints "
                          f"for {max_items} items do not fit")
    if mode == "swiglu":
        code, want = 3, torch.bfloat16
        if not w.up_tile_offset:
            raise KernelError("grouped gemm swiglu: the weight is no gated pair")
    elif mode == "store" and not w.up_tile_offset:
        code, want = (1, torch.float32) if y.dtype == torch.float32 else (0, torch.bfloat16)
    else:
        raise KernelError(f"grouped gemm: mode {mode!r} does not fit the weight")
    if y.dtype != want:
        raise KernelError(f"grouped gemm {mode}: output must be {want}, got {y.dtype}")
    name = "gemm_bf16_grouped " + label if label else "gemm_bf16_grouped"
    _check(_lib("gemm_bf16_tc2", _defines_key(_PAIR_DEFINES), _PAIR_DEFINES).jb_gemm_bf16_pair_grouped(
        _ptr(x), _ptr(w.tiles), w.n_tiles, w.up_tile_offset, _ptr(y), T, N, K, N, code, _ptr(table), int(max_items),
        gate_limit, gate_alpha, _ptr(kernel_status(x.device)), _stream()), name)


def gemm_qkv_rope_supported(T: int, hd: int) -> bool:
    """Whether the fused projection below takes this step: prompt-sized token counts and a head size that
    divides the kernel's 256 columns with half-heads of whole 16-column loads."""
    return _GEMM_PAIR and _QKV_FUSED and T >= QKV_FUSED_MIN_TOKENS and hd in (32, 64, 128, 256)


_QKV_FUSED = os.environ.get("JANUS_QKV_FUSED", "1") != "0"   # 0: projection, then rotation and cache append apart


def gemm_qkv_rope_cache(x: torch.Tensor, w: PackedWeight, q_out: torch.Tensor, cos_sin: torch.Tensor,
                        positions: torch.Tensor, dest: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                        nh: int, nkv: int, hd: int, page_size: int) -> None:
    """The stacked q/k/v projection x[T, K] . w[(nh + 2 nkv) hd, K]^T on CTA pairs with its consumers fused
    into the epilogue: q and k rotated by cos_sin[positions], q to q_out[T, nh hd], k and v to the paged
    cache at rows dest, all bfloat16 from the float32 accumulators."""
    T, K = x.shape
    _need(x, "qkv x", torch.bfloat16)
    if not isinstance(w, PackedWeight) or (w.rows, w.cols) != ((nh + 2 * nkv) * hd, K) or w.up_tile_offset:
        raise KernelError(f"qkv: a packed weight of {(nh + 2 * nkv) * hd} x {K} is needed")
    _need(q_out, "q_out", torch.bfloat16, (T, nh * hd))
    _need(cos_sin, "rope table", torch.float32)
    if cos_sin.shape[1:] != (hd // 2, 2):
        raise KernelError(f"qkv: table shape {tuple(cos_sin.shape)} does not fit head_dim {hd}")
    _need(positions, "positions", torch.int32, (T,))
    _need(dest, "cache rows", torch.int32, (T,))
    _need(k_cache, "k cache", torch.bfloat16)
    _need(v_cache, "v cache", torch.bfloat16)
    if k_cache.shape[1:] != (nkv, page_size, hd) or v_cache.shape != k_cache.shape:
        raise KernelError(f"qkv: cache shape {tuple(k_cache.shape)} is not [pages, {nkv}, {page_size}, {hd}]")
    _check(_lib("gemm_bf16_tc2", _defines_key(_PAIR_DEFINES), _PAIR_DEFINES).jb_gemm_bf16_pair_qkv_rope(
        _ptr(x), _ptr(w.tiles), w.n_tiles, T, K, _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
        _ptr(cos_sin), _ptr(positions), _ptr(dest),
        nh, nkv, hd, page_size, _ptr(kernel_status(x.device)), _stream()), "gemm_bf16_pair_qkv_rope")


# -- sampling -----------------------------------------------------------------------
def sample(logits: torch.Tensor, out_ids: torch.Tensor, temperature: float, top_k: int, top_p: float,
           repetition_penalty: float, counts: Optional[torch.Tensor], count_rows: Optional[torch.Tensor],
           seed: int, seq_ids: torch.Tensor, steps: torch.Tensor, feedback: Optional[torch.Tensor] = None) -> None:
    B, V = logits.shape
    _need(logits, "logits", torch.float32)
    _need(out_ids, "sampled ids", torch.int32, (B,))
    _need(seq_ids, "sequence ids", torch.int32, (B,))
    _need(steps, "step counters", torch.int32, (B,))
    if count_rows is not None:
        _need(count_rows, "rows' slots", torch.int32, (B,))
    if feedback is not None:
        _need(feedback, "token feedback", torch.int32)
    if counts is not None:
        _need(counts, "token counts", torch.int32)
        if counts.shape[1] != V:
            raise KernelError("sample: counts width differs from the vocabulary")
    _check(_lib("sampling").jb_sample(
        _ptr(logits), B, V, _ptr(out_ids), temperature, int(top_k), top_p,
        repetition_penalty, _ptr(counts), _ptr(count_rows),
        seed & ((1 << 64) - 1), _ptr(seq_ids), _ptr(steps), _ptr(feedback), _stream()),
        "sample")


# -- bfloat16 attention (one library per head size) -----------------------------------
ATTENTION_MAX_HEAD_DIM = 256      # every attention kernel, float32 and bfloat16
ATTENTION_BF16_MAX_GROUP = 64     # query heads per kv head of the mma.sync prompt kernel (a row tile holds 64 rows)


def _attention_lib(hd: int):
    if hd % 8 or not 8 <= hd <= 256:
        raise KernelError(f"attention_bf16: head_dim {hd} is not a multiple of 8 in [8, 256]")
    return _lib("attention_bf16", int(hd), lambda h: dict({"JB_HEAD_DIM": h}, **_ATTN_DEFINES))


def attention_bf16_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                           block_table: torch.Tensor, q_start: torch.Tensor, kv_len: torch.Tensor,
                           n_seqs: int, max_q_len: int, nh: int, nkv: int, hd: int, page_size: int,
                           window: int, scale: float, chunk: int = 0, softcap: float = 0.0,
                           sink: bool = False) -> None:
    """Causal attention of each sequence's new tokens (the last q_len positions of
    its kv_len) over its cached keys.  `chunk`, `softcap`, `sink`: as in `attention_f32`."""
    T = q.shape[0]
    _need(q, "attention q", torch.bfloat16, (T, nh * hd))
    _need(out, "attention out", torch.bfloat16, (T, nh * hd))
    _need(k_cache, "k cache", torch.bfloat16)
    _need(v_cache, "v cache", torch.bfloat16)
    _need(block_table, "block table", torch.int32)
    _need(q_start, "q_start", torch.int32, (n_seqs + 1,))
    _need(kv_len, "kv_len", torch.int32, (n_seqs,))
    if chunk or softcap or sink:
        _check(_attention_lib(hd).jb_attention_bf16_prefill_capped(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _ptr(q_start), _ptr(kv_len),
            n_seqs, max_q_len, nh, nkv, hd, page_size, block_table.shape[1], int(window), scale, int(chunk),
            float(softcap), 1.0 if sink else 0.0, _stream()), "attention_bf16_prefill")
        return
    _check(_attention_lib(hd).jb_attention_bf16_prefill(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _ptr(q_start), _ptr(kv_len),
        n_seqs, max_q_len, nh, nkv, hd, page_size, block_table.shape[1], int(window), scale,
        _stream()), "attention_bf16_prefill")


# Constants of the estimate in `decode_splits_for` (microseconds, bytes per microsecond), read off measurements
# of the decode kernel at head sizes 64 and 128 (1 to 64 sequences of 1,024 to 4,000 keys, 8 and 40 kv heads,
# 1 to 8 splits): they rank split counts, they forecast no time.
_SPLIT_CTA_US = 3.0                 # a CTA's start, its queries, its last exchange and write
_SPLIT_PAGE_US = {64: 0.6, 128: 0.85}   # a CTA alone walks a page of 64 keys in this time (head size up to 64 / above)
_SPLIT_HBM_BYTES_PER_US = 6.2e6
_SPLIT_COMBINE_US = 3.0             # the kernel that joins the splits, plus 0.05 a split
_SPLIT_SHARED_SM = 0.2              # a CTA that shares its SM with another walks its pages this much slower
_SPLIT_CHOICES = (1, 2, 3, 4, 6, 8, 12, 16, 24, 32)


def _decode_ctas_per_sm(head_dim: int, ctas: int, pages_per_cta: int) -> int:
    """CTAs of the decode kernel that share an SM: its ring of pages is picked at the launch (in step with
    `decode_stages_for` of csrc/attention_bf16.cu): three pages for large heads (two CTAs an SM at head size
    128); small heads take two pages when there are more CTAs than fit at once (five an SM at head size 64),
    five pages for few CTAs of many pages (two an SM), else three (three an SM)."""
    ld = (head_dim + 15) // 16 * 16 + 8

    def fit(stages: int) -> int:
        smem = 18 * ld * 2 + max(2 * stages * 64 * ld * 2, (4 * 16 * (head_dim + 8) + 128) * 4)
        return max(1, min(16, 228 * 1024 // (smem + 1024)))

    if head_dim > 64:
        return fit(3)
    sms = SM_COUNT_TARGET // 2
    if ctas > sms * fit(3):
        return fit(2)
    if ctas <= sms * fit(5) and pages_per_cta >= 8:
        return fit(5)
    return fit(3)


@functools.lru_cache(maxsize=4096)
def decode_splits_for(n_seqs: int, nkv_blocks: int, max_kv_len: int, page_size: int, head_dim: int = 128) -> int:
    """Splits of the key range per (sequence, kv head), from an estimate of the kernel's time for each count.

    A launch is `n_seqs * nkv_blocks * splits` CTAs of about `pages / splits` pages each; as many CTAs as fit the
    SMs run at once (a wave).  A wave takes as long as its bytes need at the memory's rate, but no less than one
    CTA needs to walk its pages (a little longer where CTAs share an SM); the waves add up, and more than one
    split costs the kernel that joins them.  So few sequences want many splits (one sequence of 2,080 keys: 16), a batch that fills the SMs wants
    none (64 sequences over 8 kv heads: 1), and a batch that overfills them a little wants its CTAs small, so
    that the last wave is short (8 sequences over 40 kv heads, 320 CTAs for 296 places: 4 splits, 62 us against
    76 us uncut).  `max_kv_len` is the bound a step was laid out for (a power of two of pages); sequences are
    taken to be three quarters of it."""
    cap_pages = max(1, (max_kv_len + page_size - 1) // page_size)
    pages = max(1, (3 * cap_pages + 3) // 4)
    base = max(1, n_seqs * nkv_blocks)
    sms = SM_COUNT_TARGET // 2
    page_us = _SPLIT_PAGE_US[64 if head_dim <= 64 else 128]
    page_bytes = page_size * head_dim * 2 * 2
    best = (float("inf"), 1)
    for splits in _SPLIT_CHOICES:
        if splits > 1 and splits > max(1, cap_pages // 2):
            break
        per = (pages + splits - 1) // splits
        ctas = base * splits
        places = sms * _decode_ctas_per_sm(head_dim, ctas, per)
        alone = _SPLIT_CTA_US + per * page_us

        def wave(n: int) -> float:      # n CTAs at once: on how many SMs, at the memory's rate or a CTA's own pace
            sharing = 1.0 + _SPLIT_SHARED_SM * ((n + sms - 1) // sms - 1)
            return max(alone * sharing, n * per * page_bytes / _SPLIT_HBM_BYTES_PER_US)

        full, rest = divmod(ctas, places)
        cost = full * wave(places) + (wave(rest) if rest else 0.0)
        if splits > 1:
            cost += _SPLIT_COMBINE_US + 0.05 * splits
        if cost < best[0] - 1e-9:
            best = (cost, splits)
    return best[1]


def attention_bf16_decode(q: Optional[torch.Tensor], k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                          block_table: torch.Tensor, kv_len: torch.Tensor, nh: int, nkv: int, hd: int,
                          page_size: int, window: int, scale: float, workspace, max_kv_len: int,
                          n_splits: Optional[int] = None, qkv: Optional[torch.Tensor] = None,
                          cos_sin: Optional[torch.Tensor] = None, dest: Optional[torch.Tensor] = None,
                          write_kv: bool = True, chunk: int = 0, softcap: float = 0.0, sink: bool = False) -> None:
    """One new token per sequence (its last position) over its cached keys.  `chunk`, `softcap`, `sink` (with `q`
    only): as in `attention_f32`.

    Either `q` (rotated bf16 queries; the cache already holds the new token), or `qkv`: the
    projection's float32 output [B, (nh + 2 nkv) hd] (or [B, nh hd] with write_kv False), which the
    kernel rotates with `cos_sin` (None: no rotation), appends to the cache at rows `dest` and uses."""
    B = out.shape[0]
    _need(out, "attention out", torch.bfloat16, (B, nh * hd))
    _need(k_cache, "k cache", torch.bfloat16)
    _need(v_cache, "v cache", torch.bfloat16)
    _need(block_table, "block table", torch.int32)
    _need(kv_len, "kv_len", torch.int32, (B,))
    n_rb = (nh // nkv + 15) // 16
    if n_splits is None:
        n_splits = decode_splits_for(B, nkv * n_rb, max_kv_len, page_size, hd)
    part_o = part_ml = None
    if n_splits > 1:
        part_o = workspace.get("attn_part_o", (B * nh * n_splits * hd,), torch.float32)
        part_ml = workspace.get("attn_part_ml", (B * nh * n_splits * 2,), torch.float32)
    lib = _attention_lib(hd)
    kernels = 2 if n_splits > 1 else 1
    if qkv is None:
        _need(q, "attention q", torch.bfloat16, (B, nh * hd))
        if chunk or softcap or sink:
            _check(lib.jb_attention_bf16_decode_capped(
                _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(block_table),
                _ptr(kv_len), B, nh, nkv, hd, page_size, block_table.shape[1], int(window), scale,
                int(n_splits), int(chunk), float(softcap), 1.0 if sink else 0.0, _stream()),
                "attention_bf16_decode", kernels=kernels)
            return
        _check(lib.jb_attention_bf16_decode(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(block_table),
            _ptr(kv_len), B, nh, nkv, hd, page_size, block_table.shape[1], int(window), scale,
            int(n_splits), _stream()), "attention_bf16_decode", kernels=kernels)
        return
    if chunk or softcap or sink:
        raise KernelError("attention decode: the kernel that rotates and appends takes no chunked mask, cap or sink")
    _need(qkv, "qkv", torch.float32)
    width = (nh + 2 * nkv) * hd if write_kv else nh * hd
    if qkv.shape[0] != B or qkv.shape[1] < width:
        raise KernelError(f"attention decode: qkv shape {tuple(qkv.shape)} does not hold {B} rows of width {width}")
    if cos_sin is not None:
        _need(cos_sin, "rope table", torch.float32)
        if cos_sin.shape[1:] != (hd // 2, 2):
            raise KernelError(f"attention decode: table shape {tuple(cos_sin.shape)} does not fit head_dim {hd}")
    if write_kv:
        _need(dest, "cache rows", torch.int32, (B,))
    _check(lib.jb_attention_bf16_decode_fused(
        _ptr(qkv), qkv.shape[1], _ptr(cos_sin), _ptr(dest), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(part_o),
        _ptr(part_ml), _ptr(block_table), _ptr(kv_len), B, nh, nkv, hd, page_size, block_table.shape[1], int(window),
        scale, int(n_splits), int(write_kv), _stream()), "attention_bf16_decode_fused", kernels=kernels)


# -- tcgen05 prefill attention (head sizes up to 256 in steps of 8, up to 128 query heads per kv head) -----
ATTENTION_TC_MAX_HEAD_DIM = 256


def attention_tc_supported(nh: int, nkv: int, hd: int) -> bool:
    g = nh // max(nkv, 1)
    return (_ATTN_TC and 0 < hd <= ATTENTION_TC_MAX_HEAD_DIM and hd % 8 == 0 and nkv > 0 and nh % nkv == 0
            and g <= 128)


def _attention_tc_row(hd: int) -> int:
    """The build that takes head size `hd`: rows of 64, 128 or 256 dims in shared memory."""
    return 64 if hd <= 64 else 128 if hd <= 128 else 256


def attention_tc_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                         block_table: torch.Tensor, q_start: torch.Tensor, kv_len: torch.Tensor,
                         n_seqs: int, max_q_len: int, nh: int, nkv: int, hd: int, page_size: int,
                         window: int, scale: float, chunk: int = 0, softcap: float = 0.0,
                         sink: bool = False) -> None:
    """As attention_bf16_prefill, on the tcgen05 tensor cores.  `chunk`, `softcap`, `sink`: as in `attention_f32`."""
    T = q.shape[0]
    _need(q, "attention q", torch.bfloat16, (T, nh * hd))
    _need(out, "attention out", torch.bfloat16, (T, nh * hd))
    _need(k_cache, "k cache", torch.bfloat16)
    _need(v_cache, "v cache", torch.bfloat16)
    _need(block_table, "block table", torch.int32)
    _need(q_start, "q_start", torch.int32, (n_seqs + 1,))
    _need(kv_len, "kv_len", torch.int32, (n_seqs,))
    if tuple(k_cache.shape[1:]) != (nkv, page_size, hd) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention_tc: cache shape {tuple(k_cache.shape)} does not fit [pages, {nkv}, {page_size}, {hd}]")
    lib = _lib("attention_tc", _attention_tc_row(hd), lambda h: dict({"JB_HEAD_DIM": h}, **_ATTN_TC_DEFINES))
    if chunk or softcap or sink:
        _check(lib.jb_attention_tc_prefill_capped(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _ptr(q_start), _ptr(kv_len),
            T, k_cache.shape[0], n_seqs, max_q_len, nh, nkv, hd, page_size, block_table.shape[1], int(window),
            scale, int(chunk), float(softcap), 1.0 if sink else 0.0, _ptr(kernel_status(q.device)), _stream()),
            "attention_tc_prefill")
        return
    _check(lib.jb_attention_tc_prefill(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _ptr(q_start), _ptr(kv_len),
        T, k_cache.shape[0], n_seqs, max_q_len, nh, nkv, hd, page_size, block_table.shape[1], int(window),
        scale, _ptr(kernel_status(q.device)), _stream()), "attention_tc_prefill")


# -- several residual streams per token -------------------------------------------------
def embed_streams(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, streams: int,
                  feedback: Optional[torch.Tensor] = None, token_slot: Optional[torch.Tensor] = None) -> None:
    """out[t, s, :] = float32(table[ids[t], :]) for every stream s (out: [T, streams * H])."""
    T = out.shape[0]
    H = out.shape[1] // streams
    _need(table, "embed table")
    _need(ids, "token ids", torch.int32, (T,))
    _need(out, "embed out", torch.float32, (T, streams * H))
    if table.shape[1] != H:
        raise KernelError(f"embed: table width {table.shape[1]} != output width {H}")
    _check(_lib("hyper").jb_embed_streams(
        _ptr(table), dtype_code(table.dtype), _ptr(ids), _ptr(out), T, H, int(streams), _ptr(feedback),
        _ptr(token_slot), _stream()), "embed_streams")


def streams_rmsnorm(x: torch.Tensor, streams: int, weights: Optional[torch.Tensor], gamma: torch.Tensor, eps: float,
                    out: torch.Tensor, row_index: Optional[torch.Tensor] = None,
                    clear: Optional[torch.Tensor] = None, clear2: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(sum_s weights[s] * x[row, s, :]) * gamma with x float32 [*, streams * H]; weights None:
    the plain sum.  `clear`: a float32 [rows, H] tensor whose rows are set to zero by the same launch; `clear2`:
    a float32 scratch tensor (whole 16-byte vectors) that it sets to zero besides."""
    rows, H = out.shape
    _need(x, "streams x", torch.float32)
    if x.dim() != 2 or x.shape[1] != streams * H:
        raise KernelError(f"streams_rmsnorm: input of shape {tuple(x.shape)} is not [*, {streams} * {H}]")
    _need(gamma, "streams gamma", None, (H,))
    _need(out, "streams out")
    if weights is not None:
        _need(weights, "stream weights", torch.float32, (streams,))
    if row_index is not None:
        _need(row_index, "streams row_index", torch.int32, (rows,))
    elif x.shape[0] < rows:
        raise KernelError("streams_rmsnorm: fewer input rows than output rows")
    if clear is not None:
        _need(clear, "streams clear", torch.float32, (rows, H))
    _check(_lib("hyper").jb_streams_rmsnorm(
        _ptr(x), _ptr(row_index), _ptr(weights), int(streams), _ptr(gamma), dtype_code(gamma.dtype), eps, _ptr(out),
        dtype_code(out.dtype), rows, H, _ptr(clear), _ptr(clear2), 0 if clear2 is None else clear2.numel(), _stream()),
        "streams_rmsnorm")


def streams_mix(x: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, out_weights: torch.Tensor, streams: int) -> None:
    """x[t, to, :] <- sum_s mix[s, to] * x[t, s, :] + out_weights[to] * y[t, :], every stream from the old ones."""
    T, H = y.shape
    _need(x, "streams x", torch.float32, (T, streams * H))
    _need(y, "sublayer output", torch.float32)
    _need(mix, "stream mix", torch.float32, (streams, streams))
    _need(out_weights, "stream out weights", torch.float32, (streams,))
    _check(_lib("hyper").jb_streams_mix(_ptr(x), _ptr(y), _ptr(mix), _ptr(out_weights), T, int(streams), H, _stream()),
           "streams_mix")


def streams_mix_rmsnorm(x: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, out_weights: torch.Tensor,
                        next_weights: torch.Tensor, streams: int, gamma: torch.Tensor, eps: float,
                        out: torch.Tensor, clear2: Optional[torch.Tensor] = None) -> None:
    """`streams_mix(x, y, mix, out_weights)` and then `streams_rmsnorm(x, next_weights, gamma) -> out` with y
    cleared, in one launch and with the same sums."""
    T, H = y.shape
    _need(x, "streams x", torch.float32, (T, streams * H))
    _need(y, "sublayer output", torch.float32)
    _need(mix, "stream mix", torch.float32, (streams, streams))
    _need(out_weights, "stream out weights", torch.float32, (streams,))
    _need(next_weights, "stream weights", torch.float32, (streams,))
    _need(gamma, "streams gamma", None, (H,))
    _need(out, "streams out", None, (T, H))
    _check(_lib("hyper").jb_streams_mix_rmsnorm(
        _ptr(x), _ptr(y), _ptr(mix), _ptr(out_weights), _ptr(next_weights), int(streams), _ptr(gamma),
        dtype_code(gamma.dtype), eps, _ptr(out), dtype_code(out.dtype), T, H, _ptr(clear2),
        0 if clear2 is None else clear2.numel(), _stream()), "streams_mix_rmsnorm")


# -- linear attention with decay ----------------------------------------------------------
LIGHTNING_SEGMENT = 128       # tokens of a segment when a long prompt's recurrence runs in segments side by side


def lightning_scan(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, out: torch.Tensor, state: torch.Tensor,
                   q_start: torch.Tensor, seq_slot: torch.Tensor, decay: torch.Tensor, n_seqs: int, heads: int,
                   dim: int, vdim: int, max_q_len: int = 1, workspace=None) -> None:
    """Per sequence and head S <- decay S + silu(k_t) silu(v_t)^T, out_t = S^T silu(q_t) over the step's tokens in
    order; proj float32 [T, ld] holds the raw q, k, v at the given columns; state float32 [slots, heads, dim, vdim].
    With a workspace, steps whose longest sequence brings more than two segments of tokens run in three passes over
    segments (their states from zero, a prefix pass, the outputs), 3 launches; else one launch."""
    T = proj.shape[0]
    _need(proj, "lightning projections", torch.float32)
    _need(out, "lightning out", torch.float32, (T, heads * vdim))
    _need(state, "lightning state", torch.float32)
    if tuple(state.shape[1:]) != (heads, dim, vdim):
        raise KernelError(f"lightning_scan: state of shape {tuple(state.shape)} is not [slots, {heads}, {dim}, {vdim}]")
    _need(q_start, "q_start", torch.int32, (n_seqs + 1,))
    _need(seq_slot, "sequence slots", torch.int32, (n_seqs,))
    _need(decay, "decay", torch.float32, (heads,))
    if max(q_col + heads * dim, k_col + heads * dim, v_col + heads * vdim) > proj.shape[1]:
        raise KernelError("lightning_scan: the projections' columns reach past the rows")
    seg, scratch = 0, None
    if workspace is not None and max_q_len > 2 * LIGHTNING_SEGMENT:
        seg = LIGHTNING_SEGMENT
        tiles = (max_q_len + seg - 1) // seg
        scratch = workspace.get("lightning_segments", (n_seqs * tiles * heads * dim * vdim,), torch.float32)
    _check(_lib("lightning").jb_lightning_scan(
        _ptr(proj), proj.shape[1], int(q_col), int(k_col), int(v_col), _ptr(out), _ptr(state), _ptr(q_start),
        _ptr(seq_slot), _ptr(decay), n_seqs, heads, dim, vdim, int(max_q_len), seg, _ptr(scratch), _stream()),
        "lightning_scan", kernels=3 if seg else 1)


def gated_rmsnorm(o: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """out = o / sqrt(mean(o^2) + eps) * weight * sigmoid(gate); o float32 [T, N], gate a float32 view [T, N] of
    rows that may be wider (its row stride is passed on)."""
    T, N = o.shape
    _need(o, "gated norm input", torch.float32)
    _need(weight, "gated norm weight", None, (N,))
    _need(out, "gated norm out", None, (T, N))
    if _checks[0] and (gate.dtype != torch.float32 or tuple(gate.shape) != (T, N) or gate.stride(1) != 1):
        raise KernelError("gated_rmsnorm: the gate must be float32 [T, N] with unit column stride")
    _check(_lib("lightning").jb_gated_rmsnorm(
        _ptr(o), _ptr(weight), dtype_code(weight.dtype), _ptr(gate), gate.stride(0), eps, _ptr(out),
        dtype_code(out.dtype), T, N, _stream()), "gated_rmsnorm")


# -- differential attention -----------------------------------------------------------------
def conv_rope_cache(proj: torch.Tensor, conv_w: Optional[torch.Tensor], taps: int, conv_state: Optional[torch.Tensor],
                    token_seq: torch.Tensor, q_start: torch.Tensor, seq_slot: torch.Tensor, positions: torch.Tensor,
                    cos_sin: Optional[torch.Tensor], rot: int, q_out: torch.Tensor, dest: torch.Tensor,
                    k_cache: torch.Tensor, v_cache: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int,
                    page_size: int, update_state: bool = False) -> None:
    """Short causal convolution over time on every channel of the projected q, k, v (float32 [T, C]), rotation of
    the first `rot` dimensions of every q and k vector, q out in float32, k and v into the paged caches.
    `update_state`: every sequence brings one token and the convolution's state takes it in the same launch."""
    T = proj.shape[0]
    C = heads * 2 * dim + kv_heads * 2 * dim + kv_heads * vdim
    _need(proj, "projections", torch.float32, (T, C))
    _need(q_out, "q out", torch.float32, (T, heads * 2 * dim))
    _need(dest, "cache rows", torch.int32, (T,))
    _need(token_seq, "token_seq", torch.int32, (T,))
    _need(positions, "positions", torch.int32, (T,))
    _need(k_cache, "k cache")
    _need(v_cache, "v cache", k_cache.dtype)
    if tuple(k_cache.shape[1:]) != (2 * kv_heads, page_size, dim) or tuple(v_cache.shape[1:]) != (kv_heads, page_size, vdim):
        raise KernelError(f"conv_rope_cache: caches of shapes {tuple(k_cache.shape)}, {tuple(v_cache.shape)} do not fit")
    if conv_w is not None:
        _need(conv_w, "conv weights", torch.float32, (C, taps))
    if conv_w is not None and taps > 1:
        _need(conv_state, "conv state", torch.float32)
        if tuple(conv_state.shape[1:]) != (taps - 1, C):
            raise KernelError(f"conv_rope_cache: state of shape {tuple(conv_state.shape)} is not [slots, {taps - 1}, {C}]")
    if cos_sin is not None:
        _need(cos_sin, "rotation table", torch.float32)
        if tuple(cos_sin.shape[1:]) != (rot // 2, 2):
            raise KernelError(f"conv_rope_cache: table of shape {tuple(cos_sin.shape)} does not fit {rot} rotated dimensions")
    _check(_lib("diff_attention").jb_conv_rope_cache(
        _ptr(proj), proj.shape[1], _ptr(conv_w), int(taps), _ptr(conv_state), int(update_state), _ptr(token_seq), _ptr(q_start),
        _ptr(seq_slot), _ptr(positions), _ptr(cos_sin), int(rot), _ptr(q_out), _ptr(dest), _ptr(k_cache), _ptr(v_cache),
        dtype_code(k_cache.dtype), T, heads, kv_heads, dim, vdim, page_size, _stream()), "conv_rope_cache")


def conv_state_update(proj: torch.Tensor, conv_state: torch.Tensor, taps: int, q_start: torch.Tensor,
                      seq_slot: torch.Tensor, n_seqs: int) -> None:
    """The convolution's state of every sequence of the step takes the last taps - 1 projected values."""
    _need(proj, "projections", torch.float32)
    _need(conv_state, "conv state", torch.float32)
    _check(_lib("diff_attention").jb_conv_state_update(
        _ptr(proj), proj.shape[1], _ptr(conv_state), int(taps), _ptr(q_start), _ptr(seq_slot), n_seqs, proj.shape[1],
        _stream()), "conv_state_update")


def diff_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                   block_table: torch.Tensor, token_seq: torch.Tensor, positions: torch.Tensor, heads: int, kv_heads: int,
                   dim: int, vdim: int, page_size: int, window: int, keep_first: int, scale: float, lam: float, eps: float,
                   out_scale: float) -> None:
    """Two softmax maps per head over the same values, o = a1 - lam a2, unit norm over the head, times out_scale."""
    T = q.shape[0]
    _need(q, "attention q", torch.float32, (T, heads * 2 * dim))
    _need(out, "attention out", k_cache.dtype, (T, heads * vdim))
    _need(k_cache, "k cache")
    _need(v_cache, "v cache", k_cache.dtype)
    _need(block_table, "block table", torch.int32)
    _need(token_seq, "token_seq", torch.int32, (T,))
    _need(positions, "positions", torch.int32, (T,))
    _check(_lib("diff_attention").jb_diff_attention(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), dtype_code(k_cache.dtype), _ptr(out), dtype_code(out.dtype),
        _ptr(block_table), _ptr(token_seq), _ptr(positions), T, heads, kv_heads, dim, vdim, page_size,
        block_table.shape[1], int(window), int(keep_first), scale, lam, eps, out_scale, _stream()), "diff_attention")


DIFF_PREFILL_MAX_GROUP = 64     # query heads per key/value head that fit a tile of the tensor-core prompt kernel


def diff_attention_prefill_supported(heads: int, kv_heads: int, dim: int, vdim: int, page_size: int) -> bool:
    """Whether the tensor-core kernel for prompt steps takes these sizes (bfloat16): key and value sizes that are
    multiples of 16 up to 128, pages of 64 keys, at most 64 query heads per key/value head."""
    return (_DIFF_MMA and dim % 16 == 0 and vdim % 16 == 0 and 16 <= dim <= 128 and 16 <= vdim <= 128
            and page_size == 64 and kv_heads > 0 and heads % kv_heads == 0 and heads // kv_heads <= DIFF_PREFILL_MAX_GROUP)


_DIFF_MMA = os.environ.get("JANUS_DIFF_MMA", "1") != "0"     # 0: prompts attend on the CUDA-core kernel
_DIFF_MMA_DEFINES = _defines_from_env("JANUS_DIFF_MMA_DEFINES")   # e.g. JB_DIFF_CTAS=1 (experiments)


def diff_attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                           block_table: torch.Tensor, q_start: torch.Tensor, kv_len: torch.Tensor, n_seqs: int,
                           max_q_len: int, heads: int, kv_heads: int, dim: int, vdim: int, page_size: int, window: int,
                           keep_first: int, scale: float, lam: float, eps: float, out_scale: float) -> None:
    """`diff_attention` for the new tokens of prompt steps (each sequence's last q_len positions of its kv_len) in
    bfloat16 on the tensor cores; one library per (dim, vdim)."""
    T = q.shape[0]
    _need(q, "attention q", torch.float32, (T, heads * 2 * dim))
    _need(out, "attention out", torch.bfloat16, (T, heads * vdim))
    _need(k_cache, "k cache", torch.bfloat16)
    _need(v_cache, "v cache", torch.bfloat16)
    _need(block_table, "block table", torch.int32)
    _need(q_start, "q_start", torch.int32, (n_seqs + 1,))
    _need(kv_len, "kv_len", torch.int32, (n_seqs,))
    lib = _lib("diff_attention_mma", (int(dim), int(vdim)), lambda k: dict({"JB_DIFF_D": k[0], "JB_DIFF_E": k[1]}, **_DIFF_MMA_DEFINES))
    _check(lib.jb_diff_attention_prefill(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _ptr(q_start), _ptr(kv_len), n_seqs,
        max_q_len, heads, kv_heads, dim, vdim, page_size, block_table.shape[1], int(window), int(keep_first), scale, lam,
        eps, out_scale, _stream()), "diff_attention_prefill")


# -- a gated activation with clamped branches; scale and soft cap -------------------------------
GELU_TANH_GATE = -1.0     # as a gated product's `limit`: the tanh form of GELU on the gate (any negative value)


def clamped_glu(gate_up: torch.Tensor, out: torch.Tensor, up_col: int, limit: float, alpha: float) -> None:
    """out[t, c] = g sigmoid(alpha g) (u + 1), g = min(gate_up[t, c], limit), u = clamp(gate_up[t, up_col + c], +-limit);
    with limit < 0 (`GELU_TANH_GATE`) out[t, c] = gelu_tanh(gate) * up, with limit 0 silu(gate) * up."""
    T, I = out.shape
    _need(gate_up, "gate/up", torch.float32)
    _need(out, "activation out")
    if gate_up.dim() != 2 or gate_up.shape[0] != T:
        raise KernelError(f"clamped_glu: input of shape {tuple(gate_up.shape)} does not hold {T} rows")
    _check(_lib("elementwise").jb_clamped_glu(_ptr(gate_up), gate_up.shape[1], int(up_col), _ptr(out),
                                              dtype_code(out.dtype), T, I, limit, alpha, _stream()), "clamped_glu")


def scale_softcap(x: torch.Tensor, scale: float, cap: float) -> None:
    """x <- cap * tanh(x * scale / cap) in place (cap <= 0: x * scale); float32."""
    _need(x, "logits", torch.float32)
    _check(_lib("elementwise").jb_scale_softcap(_ptr(x), x.numel(), scale, cap, _stream()), "scale_softcap")


def pad_rows_bf16(x: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, :K] = x[t], out[t, K:] = 0 for bfloat16 rows: the operand of a product whose width was padded."""
    T, K = x.shape
    _need(x, "rows to pad", torch.bfloat16)
    _need(out, "padded rows", torch.bfloat16)
    if out.shape[0] != T or out.shape[1] < K:
        raise KernelError(f"pad_rows: {tuple(out.shape)} does not hold {tuple(x.shape)}")
    _check(_lib("elementwise").jb_pad_rows_bf16(_ptr(x), K, _ptr(out), out.shape[1], T, _stream()), "pad_rows")


# -- a sublayer whose output is normed before it joins the residual stream ---------------------------------
def sublayer_norm_add(y: Optional[torch.Tensor], gamma: Optional[torch.Tensor], eps: float, mult: float,
                      residual: torch.Tensor, x_out: Optional[torch.Tensor],
                      clear: Optional[torch.Tensor] = None, clear2: Optional[torch.Tensor] = None) -> None:
    """residual += mult * y / sqrt(mean(y^2) + eps) * gamma (row by row; y float32, set to zero afterwards), then
    x_out = residual in x_out's dtype.  y None: the cast alone; x_out None: the sum alone.  `clear`, `clear2`: float32
    scratch tensors (whole 16-byte vectors) that the same launch sets to zero."""
    T, H = residual.shape
    _need(residual, "residual", torch.float32)
    if y is not None:
        _need(y, "sublayer output", torch.float32, (T, H))
        _need(gamma, "norm weight", None, (H,))
    if x_out is not None:
        _need(x_out, "sublayer input", None, (T, H))
    for c in (clear, clear2):
        if c is not None:
            _need(c, "buffer to clear", torch.float32)
    _check(_lib("elementwise").jb_sublayer_norm_add(
        _ptr(y), _ptr(gamma) if y is not None else None, dtype_code(gamma.dtype) if y is not None else F32, eps, mult,
        _ptr(residual), _ptr(x_out), dtype_code(x_out.dtype) if x_out is not None else F32, T, H, _ptr(clear),
        0 if clear is None else clear.numel(), _ptr(clear2), 0 if clear2 is None else clear2.numel(), _stream()),
        "sublayer_norm_add")


# -- attention mixers whose queries and keys are normed over the whole projection ----------------------------
def qk_norm_rope_cache(proj: torch.Tensor, bq: Optional[torch.Tensor], bk: Optional[torch.Tensor], wq: torch.Tensor,
                       wk: torch.Tensor, eps: float, table: Optional[torch.Tensor], rot: int, positions: torch.Tensor,
                       q_out: torch.Tensor, dest: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                       v_cache: Optional[torch.Tensor], heads: int, kv_heads: int, dim: int, page_size: int,
                       write_kv: bool = True, stored_dim: Optional[int] = None) -> None:
    """proj float32 [T, >= (heads + kv_heads) dim]: q and k as projected.  Adds the biases, appends k (with its bias,
    before norm and rotation) to the value pages, norms q and k each over its whole row, turns the first `rot`
    dimensions of every head by the table's cos and sin at the token's position, writes q [T, heads dim] and
    appends k to the key pages.  write_kv False: q alone.  `stored_dim` >= dim: the size a head has in q and in the
    pages (extra columns zero)."""
    T = q_out.shape[0]
    dp = dim if stored_dim is None else int(stored_dim)
    _need(proj, "projections", torch.float32)
    if proj.shape[0] != T:
        raise KernelError("qk_norm_rope_cache: projections and queries differ in their rows")
    _need(q_out, "q_out", None, (T, heads * dp))
    _need(wq, "q norm weight", torch.float32, (heads * dim,))
    _need(positions, "positions", torch.int32, (T,))
    if bq is not None:
        _need(bq, "q bias", torch.float32, (heads * dim,))
    if table is not None and rot > 0:
        _need(table, "rotation table", torch.float32)
        if tuple(table.shape[1:]) != (rot // 2, 2):
            raise KernelError(f"qk_norm_rope_cache: table of shape {tuple(table.shape)} does not fit {rot} dimensions")
    if write_kv:
        _need(wk, "k norm weight", torch.float32, (kv_heads * dim,))
        if bk is not None:
            _need(bk, "k bias", torch.float32, (kv_heads * dim,))
        _need(dest, "cache rows", torch.int32, (T,))
        _need(k_cache, "key pages", q_out.dtype)
        _need(v_cache, "value pages", q_out.dtype)
    _check(_lib("qk_prep").jb_qk_norm_rope_cache(
        _ptr(proj), proj.shape[1], _ptr(bq), _ptr(bk) if write_kv else None, _ptr(wq), _ptr(wk) if write_kv else None,
        eps, _ptr(table) if rot > 0 else None, int(rot), _ptr(positions), _ptr(q_out), dtype_code(q_out.dtype),
        _ptr(dest) if write_kv else None, _ptr(k_cache) if write_kv else None, _ptr(v_cache) if write_kv else None,
        T, heads, kv_heads, dim, dp, page_size, int(write_kv), _stream()), "qk_norm_rope_cache")


def latent_prep(proj: torch.Tensor, q_width: int, rank: int, weight: Optional[torch.Tensor], eps: float,
                q_out: torch.Tensor, dest: Optional[torch.Tensor], c_cache: Optional[torch.Tensor],
                write_c: bool = True, stored_rank: Optional[int] = None) -> None:
    """proj float32 [T, >= q_width (+ rank)]: q_out = the first q_width columns in q_out's dtype; the next `rank`
    columns, divided by their root mean square and multiplied by `weight`, are appended to the pages as the token's
    key row (one key head of size rank, stored in rows of `stored_rank` >= rank columns).  write_c False: the
    queries alone."""
    T = q_out.shape[0]
    rp = rank if stored_rank is None else int(stored_rank)
    _need(proj, "projections", torch.float32)
    if proj.shape[0] != T:
        raise KernelError("latent_prep: projections and queries differ in their rows")
    _need(q_out, "q_out", None, (T, q_width))
    if write_c:
        _need(weight, "latent norm weight", torch.float32, (rank,))
        _need(dest, "cache rows", torch.int32, (T,))
        _need(c_cache, "latent pages", q_out.dtype)
    _check(_lib("qk_prep").jb_latent_prep(
        _ptr(proj), proj.shape[1], int(q_width), int(rank), rp, _ptr(weight) if write_c else None, eps, _ptr(q_out),
        dtype_code(q_out.dtype), _ptr(dest) if write_c else None, _ptr(c_cache) if write_c else None, T, int(write_c),
        _stream()), "latent_prep")


# -- the selective state-space mixer ---------------------------------------------------------------------------
MAMBA2_SEGMENT = 128     # tokens of a segment when a long prompt's recurrence runs in segments side by side


@functools.lru_cache(maxsize=None)
def _sm_count() -> int:
    return torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count


def mamba2_segment_for(n_seqs: int, max_q_len: int, heads: int, n_state: int, vdim: int) -> int:
    """Tokens a segment when the recurrence of a long prompt runs in segments: a block walks one (segment, head, 64
    value columns), four blocks share an SM (two for more than 128 state rows), and the blocks run in waves; the
    length (a multiple of the 16 tokens staged at a time, 64 to 256) is the one whose waves x length is least,
    with a little for every further segment (the prefix pass walks them one after another).  2,048 tokens of 64
    heads on 148 SMs: 128 tokens make 1,024 blocks, two waves of the 592 that fit; 240 tokens make 576, one wave."""
    slots = _sm_count() * (4 if n_state <= 128 else 2)
    best, best_cost = MAMBA2_SEGMENT, None
    for seg in range(64, 257, 16):
        tiles = (max_q_len + seg - 1) // seg
        blocks = n_seqs * tiles * heads * ((vdim + 63) // 64)
        cost = ((blocks + slots - 1) // slots) * seg + 2 * tiles
        if best_cost is None or cost < best_cost:
            best, best_cost = seg, cost
    return best


def causal_conv_silu(proj: torch.Tensor, col0: int, channels: int, weight: torch.Tensor, bias: Optional[torch.Tensor],
                     taps: int, state: Optional[torch.Tensor], state_off: int, token_seq: torch.Tensor,
                     q_start: torch.Tensor, seq_slot: torch.Tensor, out: torch.Tensor, n_seqs: int,
                     update_state: bool = True, single_tokens: bool = False) -> None:
    """out[t, c] = silu(bias[c] + sum_j weight[c, j] u[t - taps + 1 + j, c]) with u the columns [col0, col0 + channels)
    of proj (float32) within each sequence; the inputs before a step's first token come from `state` (float32
    [slots, n], the convolution's [taps - 1, channels] block at offset state_off of a slot's row), which afterwards
    takes the sequence's last taps - 1 inputs: a second launch, or the same one when every sequence brings one token
    (`single_tokens`)."""
    T = proj.shape[0]
    _need(proj, "projections", torch.float32)
    _need(out, "convolution out", torch.float32, (T, channels))
    _need(weight, "convolution weight", torch.float32, (channels, taps))
    if bias is not None:
        _need(bias, "convolution bias", torch.float32, (channels,))
    if taps > 1:
        _need(state, "convolution state", torch.float32)
        if state.dim() != 2 or state_off + (taps - 1) * channels > state.shape[1]:
            raise KernelError("causal_conv_silu: the state rows do not hold the convolution's inputs")
    _need(token_seq, "token sequences", torch.int32, (T,))
    _need(q_start, "q_start", torch.int32, (n_seqs + 1,))
    _need(seq_slot, "sequence slots", torch.int32, (n_seqs,))
    if single_tokens and T != n_seqs:
        raise KernelError("causal_conv_silu: single_tokens needs one token per sequence")
    two = bool(update_state and taps > 1 and not single_tokens)
    _check(_lib("mamba2").jb_causal_conv_silu(
        _ptr(proj), proj.shape[1], int(col0), int(channels), _ptr(weight), _ptr(bias), int(taps), _ptr(state),
        state.shape[1] if state is not None else 0, int(state_off), _ptr(token_seq), _ptr(q_start), _ptr(seq_slot),
        _ptr(out), T, n_seqs, int(bool(update_state)), int(bool(single_tokens)), _stream()), "causal_conv_silu",
        kernels=2 if two else 1)


def mamba2_scan(xbc: torch.Tensor, b_col: int, c_col: int, dt_raw: torch.Tensor, dt_bias: torch.Tensor,
                a_log: torch.Tensor, d_skip: torch.Tensor, out: torch.Tensor, state: torch.Tensor, state_off: int,
                q_start: torch.Tensor, seq_slot: torch.Tensor, n_seqs: int, heads: int, groups: int, n_state: int,
                vdim: int, max_q_len: int = 1, workspace=None) -> None:
    """Per sequence and head S <- a_t S + dt_t B_t x_t^T, out_t = S^T C_t + D x_t over the step's tokens in order, with
    dt_t = softplus(dt_raw_t + dt_bias) and a_t = exp(-exp(a_log) dt_t).  xbc float32 [T, ld]: x in columns
    [0, heads vdim), B at b_col and C at c_col ([groups][n_state]); dt_raw a float32 view [T, heads] of wider rows;
    state float32 [slots, n] with the recurrence's [heads, n_state, vdim] block at offset state_off of a slot's row.
    With a workspace, steps whose longest sequence brings more than two segments of tokens run in three passes over
    segments (3 launches), else one launch."""
    T = xbc.shape[0]
    _need(xbc, "convolved x, B, C", torch.float32)
    _need(out, "scan out", torch.float32, (T, heads * vdim))
    _need(state, "scan state", torch.float32)
    if state.dim() != 2 or state_off + heads * n_state * vdim > state.shape[1]:
        raise KernelError("mamba2_scan: the state rows do not hold [heads, state, vdim]")
    if _checks[0] and (dt_raw.dtype != torch.float32 or tuple(dt_raw.shape) != (T, heads) or dt_raw.stride(1) != 1):
        raise KernelError("mamba2_scan: dt must be float32 [T, heads] with unit column stride")
    for name, t in (("dt_bias", dt_bias), ("A_log", a_log), ("D", d_skip)):
        _need(t, name, torch.float32, (heads,))
    _need(q_start, "q_start", torch.int32, (n_seqs + 1,))
    _need(seq_slot, "sequence slots", torch.int32, (n_seqs,))
    if max(heads * vdim, b_col + groups * n_state, c_col + groups * n_state) > xbc.shape[1]:
        raise KernelError("mamba2_scan: the columns reach past the rows")
    seg, scratch, seg_decay = 0, None, None
    if workspace is not None and max_q_len > 2 * MAMBA2_SEGMENT:
        seg = mamba2_segment_for(n_seqs, max_q_len, heads, n_state, vdim)
        tiles = (max_q_len + seg - 1) // seg
        scratch = workspace.get("mamba2_segments", (n_seqs * tiles * heads * n_state * vdim,), torch.float32)
        seg_decay = workspace.get("mamba2_segment_decay", (n_seqs * tiles * heads,), torch.float32)
    _check(_lib("mamba2").jb_mamba2_scan(
        _ptr(xbc), xbc.shape[1], int(b_col), int(c_col), _ptr(dt_raw), dt_raw.stride(0), _ptr(dt_bias), _ptr(a_log),
        _ptr(d_skip), _ptr(out), _ptr(state), state.shape[1], int(state_off), _ptr(q_start), _ptr(seq_slot), n_seqs,
        heads, groups, n_state, vdim, int(max_q_len), seg, _ptr(scratch), _ptr(seg_decay), _stream()),
        "mamba2_scan", kernels=3 if seg else 1)


def gated_group_rmsnorm(y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, parts: int,
                        out: torch.Tensor) -> None:
    """out = (y * silu(gate)) divided, within each of `parts` equal pieces of a row, by the piece's root mean square
    (eps inside the root), times weight; y float32 [T, N], gate a float32 view [T, N] of rows that may be wider."""
    T, N = y.shape
    _need(y, "gated norm input", torch.float32)
    _need(weight, "gated norm weight", torch.float32, (N,))
    _need(out, "gated norm out", None, (T, N))
    if _checks[0] and (gate.dtype != torch.float32 or tuple(gate.shape) != (T, N) or gate.stride(1) != 1):
        raise KernelError("gated_group_rmsnorm: the gate must be float32 [T, N] with unit column stride")
    _check(_lib("mamba2").jb_gated_group_rmsnorm(
        _ptr(y), _ptr(gate), gate.stride(0), _ptr(weight), eps, _ptr(out), dtype_code(out.dtype), T, N, int(parts),
        _stream()), "gated_group_rmsnorm")


# -- layer norm, scaled sums into the residual stream, sublayers of two branches ---------------------------------
def join_norm(stream: torch.Tensor, ya: Optional[torch.Tensor] = None, yb: Optional[torch.Tensor] = None,
              wa: Optional[torch.Tensor] = None, wb: Optional[torch.Tensor] = None, mult: float = 1.0,
              mult_b: Optional[float] = None, scale: Optional[torch.Tensor] = None, extra: Optional[torch.Tensor] = None,
              gamma: Optional[torch.Tensor] = None, eps: float = 0.0, center: bool = True,
              x_out: Optional[torch.Tensor] = None, row_index: Optional[torch.Tensor] = None,
              clear: Optional[torch.Tensor] = None, clear2: Optional[torch.Tensor] = None) -> None:
    """One launch, row by row of the float32 stream r [T, W], every step optional:
    y = ya, or with branch weights y = mult ya / rms(ya) wa + mult_b yb / rms(yb) wb (mult_b None: mult), or with two
    branches and no branch weights y = mult ya + mult_b yb; r += scale * y (ya, yb set to zero);
    r += extra; x_out = norm(r) * gamma (center: layer norm without bias, else root mean square), eps inside the
    roots.  With `row_index` x_out's rows are norm(r[row_index[i]]) and r is only read.  `clear`, `clear2`: float32
    scratch tensors (whole 16-byte vectors) set to zero on the way."""
    W = stream.shape[1]
    T = stream.shape[0] if row_index is None else row_index.shape[0]
    _need(stream, "stream", torch.float32)
    for t, name in ((ya, "sublayer output"), (yb, "second branch"), (extra, "stream to add")):
        if t is not None:
            _need(t, name, torch.float32, tuple(stream.shape))
    for t, name in ((wa, "branch weight"), (wb, "branch weight"), (scale, "scale"), (gamma, "norm weight")):
        if t is not None:
            _need(t, name, torch.float32, (W,))
    if x_out is not None:
        _need(x_out, "normed rows", None, (T, W))
    if row_index is not None:
        _need(row_index, "row index", torch.int32)
    for c in (clear, clear2):
        if c is not None:
            _need(c, "buffer to clear", torch.float32)
    _check(_lib("layer_norm").jb_join_norm(
        _ptr(stream), _ptr(ya), _ptr(yb), _ptr(wa), _ptr(wb), float(mult), float(mult if mult_b is None else mult_b),
        _ptr(scale), _ptr(extra), _ptr(gamma),
        float(eps), int(bool(center)), _ptr(x_out), dtype_code(x_out.dtype) if x_out is not None else F32,
        _ptr(row_index), T, W, _ptr(clear), 0 if clear is None else clear.numel(), _ptr(clear2),
        0 if clear2 is None else clear2.numel(), _stream()), "join_norm")


def head_norm_gate(o: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
                   heads: int, e: int, sigmoid: bool = False, denom: Optional[torch.Tensor] = None) -> None:
    """out[t, h] = o[t, h] / sqrt(mean(o[t, h]^2) + eps) * weight * act(gate[t, h]) for float32 o [T, heads e], a float32
    gate (a view whose rows may be wider) and a weight [e] that the heads share or [heads e] with a part for every
    head; act is SiLU, or the sigmoid.  `denom` (float32 [T, heads]): o[t, h] is first divided by denom[t, h]."""
    T = o.shape[0]
    _need(o, "head outputs", torch.float32, (T, heads * e))
    per_head = weight.numel() == heads * e and heads > 1
    _need(weight, "head norm weight", torch.float32, (heads * e,) if per_head else (e,))
    if denom is not None:
        _need(denom, "divisors", torch.float32, (T, heads))
    _need(out, "gated heads", None, (T, heads * e))
    if gate.dtype != torch.float32 or gate.stride(1) != 1 or gate.shape != o.shape:
        raise KernelError("head_norm_gate: the gate must be float32 columns of the heads' shape")
    _check(_lib("layer_norm").jb_head_norm_gate(_ptr(o), _ptr(gate), gate.stride(0), _ptr(weight), e if per_head else 0,
                                                _ptr(denom), float(eps), 1 if sigmoid else 0, _ptr(out), dtype_code(out.dtype), T, heads, e,
                                                _stream()), "head_norm_gate")


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, heads: int, e: int, stored: int) -> None:
    """x[t, h, j] *= sigmoid(gate[t, h, j]) in place for j < e; x [T, heads stored] holds heads of `stored` >= e numbers,
    gate: float32 columns [T, heads e] (a view whose rows may be wider)."""
    T = x.shape[0]
    _need(x, "rows to gate", None, (T, heads * stored))
    if gate.dtype != torch.float32 or gate.stride(1) != 1 or tuple(gate.shape) != (T, heads * e):
        raise KernelError("sigmoid_gate: the gate must be float32 columns, one for each number of the heads")
    _check(_lib("layer_norm").jb_sigmoid_gate(_ptr(x), dtype_code(x.dtype), _ptr(gate), gate.stride(0), T, heads, e,
                                              stored, _stream()), "sigmoid_gate")


def head_norm_rope_cache(proj: torch.Tensor, wq: Optional[torch.Tensor], wk: Optional[torch.Tensor], eps: float,
                         table: Optional[torch.Tensor], rot: int, positions: torch.Tensor, q_out: torch.Tensor,
                         dest: Optional[torch.Tensor], k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                         heads: int, kv_heads: int, dim: int, vdim: int, stored_dim: int, page_size: int,
                         write_kv: bool = True, unit_norm: bool = False, temp_coef: float = 0.0,
                         temp_every: int = 0) -> None:
    """proj float32 [T, >= heads dim + kv_heads (dim + vdim)]: q, k and v as projected.  Every head of q and k is
    divided by its own root mean square and multiplied by the weight [dim] that the heads share (None: no norm), its
    first `rot` dimensions are turned by the table's cos and sin at the token's position; q is written
    [T, heads stored_dim], k and v are appended to pages whose rows hold stored_dim numbers.  `unit_norm`: without
    weights the heads are still divided by their root mean square.  `temp_every` > 0: q is multiplied by
    1 + temp_coef ln(floor((position + 1) / temp_every) + 1)."""
    T = q_out.shape[0]
    _need(proj, "projections", torch.float32)
    if proj.shape[0] != T:
        raise KernelError("head_norm_rope_cache: projections and queries differ in their rows")
    _need(q_out, "q_out", None, (T, heads * stored_dim))
    _need(positions, "positions", torch.int32, (T,))
    for w in (wq, wk):
        if w is not None:
            _need(w, "head norm weight", torch.float32, (dim,))
    if table is not None and rot > 0:
        _need(table, "rotation table", torch.float32)
        if tuple(table.shape[1:]) != (rot // 2, 2):
            raise KernelError(f"head_norm_rope_cache: table of shape {tuple(table.shape)} does not fit {rot} dimensions")
    if write_kv:
        _need(dest, "cache rows", torch.int32, (T,))
        _need(k_cache, "key pages", q_out.dtype)
        _need(v_cache, "value pages", q_out.dtype)
    _check(_lib("qk_prep").jb_head_norm_rope_cache(
        _ptr(proj), proj.shape[1], _ptr(wq), _ptr(wk), float(eps), _ptr(table) if rot > 0 else None, int(rot),
        _ptr(positions), _ptr(q_out), dtype_code(q_out.dtype), _ptr(dest) if write_kv else None,
        _ptr(k_cache) if write_kv else None, _ptr(v_cache) if write_kv else None, T, heads, kv_heads, dim, vdim,
        stored_dim, page_size, int(write_kv), int(bool(unit_norm)), float(temp_coef), int(temp_every), _stream()),
        "head_norm_rope_cache")


# -- the gated delta rule ------------------------------------------------------------------------------------------
def delta_rule(conv: torch.Tensor, q_col: int, k_col: int, v_col: int, raw: torch.Tensor, b_col: int, a_col: int,
               a_log: torch.Tensor, dt_bias: torch.Tensor, unit_eps: float, out: torch.Tensor, state: torch.Tensor,
               state_off: int, q_start: torch.Tensor, seq_slot: torch.Tensor, n_seqs: int, heads: int, kv_heads: int,
               dim: int, vdim: int) -> None:
    """The recurrence S <- g S; w = beta (v - S^T k); S <- S + k w^T; o = S^T q per head, over each sequence's tokens
    from the state its slot holds (float32 [slots, n], the [heads, dim, vdim] block at state_off), which is updated.
    q, k (unit vectors are made here; q also times dim^-1/2) and v are columns of `conv`, beta's and the decay's
    arguments columns of `raw`; g = exp(-exp(a_log) softplus(a + dt_bias)), beta = sigmoid(b)."""
    T = conv.shape[0]
    _need(conv, "convolved projections", torch.float32)
    _need(raw, "projections", torch.float32)
    _need(out, "recurrence out", torch.float32, (T, heads * vdim))
    _need(a_log, "A_log", torch.float32, (heads,))
    _need(dt_bias, "dt_bias", torch.float32, (heads,))
    _need(state, "state", torch.float32)
    if state.dim() != 2 or state_off + heads * dim * vdim > state.shape[1]:
        raise KernelError("delta_rule: the state rows do not hold the recurrence's state")
    _need(q_start, "q_start", torch.int32, (n_seqs + 1,))
    _need(seq_slot, "sequence slots", torch.int32, (n_seqs,))
    _check(_lib("delta_rule").jb_delta_rule(
        _ptr(conv), conv.shape[1], int(q_col), int(k_col), int(v_col), _ptr(raw), raw.shape[1], int(b_col), int(a_col),
        _ptr(a_log), _ptr(dt_bias), float(unit_eps), _ptr(out), _ptr(state), state.shape[1], int(state_off),
        _ptr(q_start), _ptr(seq_slot), n_seqs, heads, kv_heads, dim, vdim, _stream()), "delta_rule")


# -- experts of which a token uses a few ---------------------------------------------------------------------------
def route_topk(logits: torch.Tensor, top: int, sel_e: torch.Tensor, sel_w: torch.Tensor, softmax: bool = False,
               groups: int = 0, keep: int = 0, experts: Optional[int] = None) -> None:
    """Per row of the float32 logits [T, >= E] (the first `experts` columns; None: all): the `top` largest (the lower
    index wins a tie) as indices (int32 [T, top]) and their scores as weights (float32 [T, top]): the logits' sigmoids,
    or with `softmax` the softmax over all experts.  `groups` > 0: the experts form that many equal groups of
    neighbours, and only experts of the `keep` groups whose best expert scores highest can be chosen."""
    T, ld = logits.shape
    E = ld if experts is None else int(experts)
    _need(logits, "router logits", torch.float32)
    _need(sel_e, "chosen experts", torch.int32, (T, top))
    _need(sel_w, "experts' weights", torch.float32, (T, top))
    if E > ld:
        raise KernelError(f"route_topk: {E} experts in rows of {ld} logits")
    _check(_lib("routed").jb_route_topk(_ptr(logits), ld, E, int(top), _ptr(sel_e), _ptr(sel_w), T,
                                        int(bool(softmax)), int(groups), int(keep), _stream()), "route_topk")


def experts_few_tokens(h: torch.Tensor, sel_e: torch.Tensor, sel_w: torch.Tensor, w_gate: torch.Tensor,
                       w_up: torch.Tensor, w_down: torch.Tensor, act: torch.Tensor, out: torch.Tensor,
                       gate_limit: float = 0.0, gate_alpha: float = 1.0, weight_on_output: bool = False) -> None:
    """out[t] += sum over the token's chosen experts e of Wd_e (act(Wg_e x) * (Wu_e x)) with x = weight * h[t] (or,
    with `weight_on_output`, of weight * Wd_e (act(Wg_e h[t]) * (Wu_e h[t]))); an
    expert's rows are streamed once for up to four of the tokens that chose it (an expert nobody chose is not read),
    sums in float32.  w_gate, w_up [E, F, W], w_down
    [E, W, F] in h's dtype; act: float32 scratch [T top, F]; out float32 [T, W]."""
    T, W = h.shape
    E, F, _ = w_gate.shape
    top = sel_e.shape[1]
    _need(h, "expert input")
    _need(w_gate, "experts' gate", h.dtype, (E, F, W))
    _need(w_up, "experts' up", h.dtype, (E, F, W))
    _need(w_down, "experts' down", h.dtype, (E, W, F))
    _need(sel_e, "chosen experts", torch.int32, (T, top))
    _need(sel_w, "experts' weights", torch.float32, (T, top))
    _need(act, "experts' scratch", torch.float32, (T * top, F))
    _need(out, "experts' out", torch.float32, (T, W))
    _check(_lib("routed").jb_experts_few_tokens(
        _ptr(h), dtype_code(h.dtype), _ptr(sel_e), _ptr(sel_w), top, _ptr(w_gate), _ptr(w_up), _ptr(w_down),
        dtype_code(w_gate.dtype), _ptr(act), _ptr(out), T, W, F, E, float(gate_limit), float(gate_alpha),
        int(bool(weight_on_output)), _stream()), "experts_few_tokens", kernels=2)


EXPERT_PLAN_MAX_EXPERTS = 1024


def expert_plan(sel_e: torch.Tensor, experts: int, F: int, W: int, order: torch.Tensor, where: torch.Tensor,
                gate_up_table: torch.Tensor, down_table: torch.Tensor) -> None:
    """Sorts the (token, choice) pairs by expert on the device (order[place] = pair, where[pair] = place) and writes
    the tile tables of the two grouped products (`gemm_bf16_grouped`): gate/up over stacks of F rows per expert in
    tiles of 128 features, down over stacks of W rows per expert in tiles of 256."""
    pairs = sel_e.numel()
    _need(sel_e, "router's choice", torch.int32)
    _need(order, "pair order", torch.int32, (pairs,))
    _need(where, "pair places", torch.int32, (pairs,))
    _need(gate_up_table, "gate/up table", torch.int32)
    _need(down_table, "down table", torch.int32)
    if (gate_up_table.numel() < 4 + 4 * grouped_max_items(pairs, experts, F, "swiglu")
            or down_table.numel() < 4 + 4 * grouped_max_items(pairs, experts, W, "store")):
        raise KernelError("expert_plan: a table is too small")
    _check(_lib("routed").jb_expert_plan(_ptr(sel_e), pairs, int(experts), int(F), int(W), _ptr(order), _ptr(where),
                                         _ptr(gate_up_table), _ptr(down_table), _stream()), "expert_plan")


def expert_gather(h: torch.Tensor, order: torch.Tensor, sel_w: Optional[torch.Tensor], top: int,
                  rows: torch.Tensor) -> None:
    """rows[i] = weight[order[i]] * h[order[i] // top] (no weights: the rows themselves): the (token, choice) pairs in
    the order the experts' products take them."""
    pairs, W = rows.shape
    _need(h, "expert input", rows.dtype)
    _need(rows, "gathered rows")
    _need(order, "pair order", torch.int32, (pairs,))
    if sel_w is not None:
        _need(sel_w, "experts' weights", torch.float32)
    _check(_lib("routed").jb_expert_gather(_ptr(h), dtype_code(h.dtype), _ptr(order), _ptr(sel_w), int(top), _ptr(rows),
                                           pairs, W, _stream()), "expert_gather")


def expert_scatter(results: torch.Tensor, where: torch.Tensor, top: int, out: torch.Tensor,
                   weights: Optional[torch.Tensor] = None) -> None:
    """out[t] += sum_k weights[t, k] results[where[t * top + k]] (float32; no weights: the plain sum)."""
    T, W = out.shape
    _need(results, "experts' results", torch.float32)
    _need(where, "pair places", torch.int32, (T * top,))
    _need(out, "experts' out", torch.float32)
    if weights is not None:
        _need(weights, "experts' weights", torch.float32, (T, top))
    _check(_lib("routed").jb_expert_scatter(_ptr(results), _ptr(where), _ptr(weights), int(top), _ptr(out), T, W,
                                            _stream()), "expert_scatter")


def scale_rows_sigmoid(x: torch.Tensor, gate: torch.Tensor) -> None:
    """x[t] *= sigmoid(gate[t]) in place: one number per row, from a float32 column (a view with a row stride)."""
    T, N = x.shape
    _need(x, "rows to scale")
    if gate.dtype != torch.float32 or gate.shape[0] != T or gate.dim() != 1:
        raise KernelError("scale_rows_sigmoid: the gate must be a float32 column with one number per row")
    _check(_lib("elementwise").jb_scale_rows_sigmoid(_ptr(x), dtype_code(x.dtype), _ptr(gate), gate.stride(0), T, N,
                                                     _stream()), "scale_rows_sigmoid")


# -- linear attention with gates that depend on the token --------------------------------------------------------
GATED_LINEAR_SEGMENT = 128


def gla_decay(proj: torch.Tensor, low_col: int, rank: int, a2t: torch.Tensor, bias: torch.Tensor, tau: float,
              alpha: torch.Tensor) -> None:
    """alpha[t, c] = sigmoid(z)^(1 / tau) with z = bias[c] + sum_j a2t[j, c] proj[t, low_col + j], in float32: the
    decays per key channel of gated linear attention from the low-rank projection's output."""
    T, C = alpha.shape
    _need(proj, "projections", torch.float32)
    _need(a2t, "second decay matrix, transposed", torch.float32, (rank, C))
    _need(bias, "decay bias", torch.float32, (C,))
    _need(alpha, "decays", torch.float32)
    if proj.shape[0] != T or low_col + rank > proj.shape[1]:
        raise KernelError("gla_decay: the projections do not hold the low-rank columns")
    _check(_lib("gated_linear").jb_gla_decay(_ptr(proj), proj.shape[1], int(low_col), int(rank), _ptr(a2t), _ptr(bias),
                                             1.0 / float(tau), _ptr(alpha), C, T, _stream()), "gla_decay")


def exp_gates(proj: torch.Tensor, i_col: int, f_col: int, bias_i: torch.Tensor, bias_f: torch.Tensor, cap: float,
              gates: torch.Tensor, state: torch.Tensor, m_off: int, q_start: torch.Tensor, seq_slot: torch.Tensor,
              n_seqs: int, heads: int) -> None:
    """Exponential gates with a running maximum per sequence and head: with i = cap tanh((zi + bi) / cap),
    f = logsigmoid(cap tanh((zf + bf) / cap)) and m_t = max(f + m_(t-1), i), gates[t, h] = (exp(f + m_(t-1) - m_t),
    exp(i - m_t), exp(-m_t), 0).  zi, zf are columns i_col + h, f_col + h of `proj`; m lives at state[slot, m_off + h]."""
    T = proj.shape[0]
    _need(proj, "projections", torch.float32)
    _need(gates, "gates", torch.float32, (T, heads, 4))
    _need(bias_i, "input gate bias", torch.float32, (heads,))
    _need(bias_f, "forget gate bias", torch.float32, (heads,))
    _need(state, "state", torch.float32)
    _need(q_start, "q_start", torch.int32, (n_seqs + 1,))
    _need(seq_slot, "sequence slots", torch.int32, (n_seqs,))
    if state.dim() != 2 or m_off + heads > state.shape[1] or max(i_col, f_col) + heads > proj.shape[1]:
        raise KernelError("exp_gates: the state rows or the projections do not hold the gates' numbers")
    _check(_lib("gated_linear").jb_exp_gates(_ptr(proj), proj.shape[1], int(i_col), int(f_col), _ptr(bias_i),
                                             _ptr(bias_f), float(cap), _ptr(gates), _ptr(state), state.shape[1],
                                             int(m_off), _ptr(q_start), _ptr(seq_slot), n_seqs, heads, _stream()),
           "exp_gates")


def gated_linear_scan(proj: torch.Tensor, q_col: int, k_col: int, v_col: int, q_scale: float, decays: torch.Tensor,
                      out: torch.Tensor, state: torch.Tensor, q_start: torch.Tensor, seq_slot: torch.Tensor,
                      n_seqs: int, heads: int, dim: int, vdim: int, max_q_len: int = 1, workspace=None,
                      divisors: Optional[torch.Tensor] = None) -> None:
    """Per sequence and head S <- diag(a_t) S + b_t k_t v_t^T, out_t = S^T (q_t q_scale) over the step's tokens in
    order; proj float32 [T, ld] holds q, k, v at the given columns.  Without `divisors`, `decays` is float32
    [T, heads dim], a decay per key channel, b = 1, and a slot's state row holds [heads, dim, vdim].  With `divisors`
    (float32 [T, heads], written), `decays` is what `exp_gates` left ([T, heads, 4]: a_t and b_t one number a head),
    a normalizer n <- a_t n + b_t k_t walks along, divisors[t, h] = max(|n . q|, exp(-m_t)) + 1e-6, and a slot's state
    row holds per head [dim, vdim] then [dim] of n.  With a workspace, steps whose longest sequence brings more than
    256 tokens run in passes over segments of 64 to 256 tokens (4 launches); else one launch."""
    T = proj.shape[0]
    scalar = divisors is not None
    _need(proj, "projections", torch.float32)
    _need(out, "recurrence out", torch.float32, (T, heads * vdim))
    _need(state, "state", torch.float32)
    _need(decays, "decays", torch.float32, (T, heads, 4) if scalar else (T, heads * dim))
    if scalar:
        _need(divisors, "divisors", torch.float32, (T, heads))
    per_head = dim * (vdim + (1 if scalar else 0))
    if state.dim() != 2 or heads * per_head > state.shape[1]:
        raise KernelError("gated_linear_scan: the state rows do not hold the recurrence's state")
    _need(q_start, "q_start", torch.int32, (n_seqs + 1,))
    _need(seq_slot, "sequence slots", torch.int32, (n_seqs,))
    if max(q_col + heads * dim, k_col + heads * dim, v_col + heads * vdim) > proj.shape[1]:
        raise KernelError("gated_linear_scan: the projections' columns reach past the rows")
    seg, scratch, seg_decay = 0, None, None
    if workspace is not None and max_q_len > 2 * GATED_LINEAR_SEGMENT:
        # the blocks are laid out as the state-space recurrence's (a segment, a head, 64 value columns; four blocks an SM
        # up to 128 rows of state, else two): the segment length that fills the SMs in whole waves is picked the same way
        seg = mamba2_segment_for(n_seqs, max_q_len, heads, dim, vdim)
        tiles = (max_q_len + seg - 1) // seg
        scratch = workspace.get("gated_linear_segments", (n_seqs * tiles * heads * per_head,), torch.float32)
        seg_decay = workspace.get("gated_linear_segment_decays", (n_seqs * tiles * heads * (1 if scalar else dim),),
                                  torch.float32)
    _check(_lib("gated_linear").jb_gated_linear_scan(
        _ptr(proj), proj.shape[1], int(q_col), int(k_col), int(v_col), float(q_scale), _ptr(decays),
        0 if scalar else heads * dim, int(scalar), _ptr(out), _ptr(divisors), _ptr(state), state.shape[1],
        _ptr(q_start), _ptr(seq_slot), n_seqs, heads, dim, vdim, int(max_q_len), seg, _ptr(scratch), _ptr(seg_decay),
        _stream()), "gated_linear_scan", kernels=4 if seg else 1)
