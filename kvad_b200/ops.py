"""Python face of the CUDA kernels.

One `Ops` object serves one compute dtype (float32 or bfloat16).  Its methods
check what the kernels assume (device, dtype, contiguity, sizes), pass raw
pointers and the current CUDA stream to the C entry points, and raise
`KernelError` with the kernel's own message when an entry point refuses.
Tensors are torch tensors only as owners of device memory; no torch operator
computes anything here, and nothing falls back to the CPU.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Optional

import torch

from .csrc import build

F32, BF16 = 0, 1
EPILOGUES = {"store": 0, "gelu_tanh": 1, "gelu_erf": 2, "residual": 3, "store_f32": 4}


class KernelError(RuntimeError):
    pass


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kvad_b200 kernels compute in float32 or bfloat16, not {dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


_SIGNATURES = {
    "rows": {
        "kvad_embed": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "kvad_layernorm": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p],
        "kvad_kv_store": [c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                          c_int, c_int, c_int, c_int, c_void_p],
        "kvad_zero_bytes": [c_void_p, c_int64, c_void_p],
    },
    "linear_simt": {
        "kvad_linear_simt": [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_int,
                             c_int, c_void_p],
    },
    "linear_tcgen05": {
        "kvad_linear_tcgen05": [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_int,
                                c_int, c_int, c_void_p],
        "kvad_linear_tcgen05_status": [],
        "kvad_linear_tcgen05_grouped": [c_void_p, c_int64, c_void_p, c_int, c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    },
    "linear_rows": {
        "kvad_linear_rows": [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_int, c_int,
                             c_void_p],
    },
    "linear_rows_f32": {
        "kvad_linear_rows": [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_int, c_int,
                             c_void_p],
    },
    "attention_simt": {
        "kvad_attention_simt": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "kvad_attention_tiled": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    },
    "attention_prefill": {
        "kvad_attention_prefill": [c_void_p, c_int64, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                   c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                   c_void_p],
    },
    "attention_decode": {
        "kvad_attention_decode_step": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int,
                                       c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "kvad_attention_decode_pre": [c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_void_p, c_int64],
        "kvad_attention_decode_takes_pre": [c_int, c_int, c_int],
    },
    "norm_rotary": {
        "kvad_rmsnorm": [c_int, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int64, c_int, c_int, c_float,
                         c_void_p],
        "kvad_residual_rmsnorm": [c_int, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int64,
                                  c_int, c_int, c_float, c_void_p],
        "kvad_scale_add": [c_void_p, c_void_p, c_float, c_int64, c_void_p],
        "kvad_rotary": [c_int, c_void_p, c_int64, c_int, c_int, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_int, c_int,
                        c_int, c_int, c_int, c_void_p, c_int64, c_void_p],
        "kvad_postnorm_rmsnorm": [c_int, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int64,
                                  c_int, c_int, c_float, c_void_p],
        "kvad_head_gate": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_void_p],
        "kvad_stream_concat": [c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "kvad_gate_mul": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_void_p],
        "kvad_cast_rows": [c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p],
        "kvad_pair_norm_sum": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_void_p],
        "kvad_tanh_cap": [c_void_p, c_int64, c_float, c_void_p],
    },
    "attention_scored": {
        "kvad_attention_scored": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                                  c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                  c_float, c_float, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p],
        "kvad_scored_merge_diff": [c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int64, c_float, c_float, c_float, c_void_p],
        "kvad_norm_turn_store": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int,
                                 c_float, c_void_p, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                                 c_int, c_int, c_int, c_int, c_int, c_void_p],
        "kvad_diff_combine": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_void_p],
        "kvad_kv_store_blend": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_void_p, c_void_p,
                                c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "kvad_turn_store": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p,
                            c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "kvad_linear_heads": [c_int, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "kvad_latent_store": [c_int, c_void_p, c_int64, c_void_p, c_int, c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                              c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    },
    "retention": {
        "kvad_retention": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                           c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                           c_int, c_float, c_float, c_int, c_int, c_int, c_void_p],
        "kvad_retention_needs_raw": [c_int, c_int],
        "kvad_row_norm_gate": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_float, c_void_p],
    },
    "gated_recurrence": {
        "kvad_gated_recurrence": [c_int, c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64,
                                  c_void_p, c_void_p, c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int,
                                  c_int, c_int, c_float, c_float, c_int, c_void_p],
        "kvad_gated_recurrence_state": [c_int, c_int, c_int, c_int],
        "kvad_decay_gate": [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "kvad_short_conv": [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p],
        "kvad_conv_state": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "kvad_head_norm_gate": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p, c_int64, c_int, c_int, c_int,
                                c_float, c_void_p],
    },
    "moe": {
        "kvad_moe_tile_rows": [],
        "kvad_moe_route_apart_rows": [],
        "kvad_moe_route": [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p],
        "kvad_moe_sort": [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p,
                          c_int, c_void_p, c_int, c_void_p],
        "kvad_relu_squared": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_void_p],
        "kvad_gather_rows": [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p],
        "kvad_grouped_linear": [c_int, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                                c_int, c_int, c_int, c_int, c_void_p],
        "kvad_clamped_glu": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_float, c_float, c_void_p],
        "kvad_scaled_glu": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "kvad_moe_combine": [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int64, c_void_p],
    },
    "channel_recurrence": {
        "kvad_residual_conv": [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                               c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "kvad_conv_keep": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
        "kvad_min_gru": [c_int, c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_void_p,
                         c_int, c_int, c_int, c_void_p],
    },
    "sampling": {
        "kvad_sample": [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "kvad_argmax": [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p],
    },
}

_bound: dict[str, ctypes.CDLL] = {}
_pdl = os.environ.get("KVAD_PDL", "1") != "0"
_switch_epoch = 0          # bumped by every switch that changes which kernels a step launches


def register_kernels(name: str, source: str, signatures: dict) -> None:
    """The door for a part that brings a kernel of its own: `source` is a `.cu` file anywhere (it may
    include this package's `common.cuh`; it must contain `KVAD_DEFINE_LAST_ERROR()` once), `signatures`
    maps its exported C entry points (returning 0 or a negative code, message through
    `kvad_last_error`) to their ctypes argument lists.  Afterwards `lib(name)` compiles it for
    sm_100a on first use and loads it like the package's own libraries; `launch(handle, status)`
    turns a refusal into a `KernelError` and counts the launch."""
    if name in _SIGNATURES and name not in build.registered_sources():
        raise ValueError(f"`{name}` is one of the package's own kernel libraries")
    build.register_source(name, source)
    _SIGNATURES[name] = dict(signatures)
    _bound.pop(name, None)


def switches_changed() -> None:
    """Called by every switch that changes which kernels a step launches: captured step graphs are
    keyed by the epoch, so a step captured under the old setting is not replayed under the new one."""
    global _switch_epoch
    _switch_epoch += 1


def switch_epoch() -> int:
    return _switch_epoch


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for every kernel of the library: a kernel may start (set up,
    fetch its weights) while the one before it in the stream still runs.  On by default; KVAD_PDL=0
    or set_pdl(False) launches plainly."""
    global _pdl
    _pdl = bool(on)
    switches_changed()
    for handle in _bound.values():
        handle.kvad_set_pdl(int(_pdl))


def lib(name: str) -> ctypes.CDLL:
    """The loaded kernel library `name` with its entry points typed."""
    hit = _bound.get(name)
    if hit is not None:
        return hit
    handle = build.load(name)
    for fn, argtypes in _SIGNATURES[name].items():
        f = getattr(handle, fn)
        f.argtypes = argtypes
        f.restype = c_int
    handle.kvad_set_pdl.argtypes = [c_int]
    handle.kvad_set_pdl.restype = None
    handle.kvad_set_pdl(int(_pdl))
    _bound[name] = handle
    return handle


#: kernel libraries by what needs them: every model ("base"), and the families a part names in `Part.kernel_families`
_FAMILY_LIBRARIES = {
    "base": {"any": ("rows", "linear_simt", "sampling"), torch.bfloat16: ("linear_rows", "linear_tcgen05"), torch.float32: ("linear_rows_f32",)},
    "causal_attention": {"any": ("attention_simt", "attention_decode"), torch.bfloat16: ("attention_prefill",), torch.float32: ()},
    "norm_rotary": {"any": ("norm_rotary",)},
    "scored_attention": {"any": ("attention_scored",)},
    "prompt_attention": {torch.bfloat16: ("attention_prefill",)},
    "retention": {"any": ("retention",)},
    "gated_recurrence": {"any": ("gated_recurrence",)},
    "moe": {"any": ("moe",)},
    "channel_recurrence": {"any": ("channel_recurrence",)},
}


def libraries_for(dtype: torch.dtype, families=None) -> list[str]:
    """Which kernel libraries a model of this compute dtype loads.  `families`: what the model's parts
    name (`Part.kernel_families`); None: a model of plain causal attention layers."""
    names: list[str] = []
    for fam in ["base", *(families if families is not None else ["causal_attention"])]:
        table = _FAMILY_LIBRARIES[fam]
        for n in (*table.get("any", ()), *table.get(dtype, ())):
            if n in build.sources() and n not in names:
                names.append(n)
    return names


_launches = 0


def launch_count() -> int:
    """How many kernels of this library have been launched (or captured into a graph) so far."""
    return _launches


def launch(handle: ctypes.CDLL, status: int) -> None:
    """For kernels registered from outside: raises the entry point's own message on a refusal, counts the launch."""
    _check(status, handle)


def stream_ptr() -> c_void_p:
    """The current CUDA stream as the entry points take it."""
    return _stream()


_sm_counts: dict[int, int] = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (asked once per device)."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    n = _sm_counts.get(idx)
    if n is None:
        n = _sm_counts[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return n


def _check(status: int, handle: ctypes.CDLL) -> None:
    global _launches
    if status != 0:
        raise KernelError(handle.kvad_last_error().decode("utf-8", "replace"))
    _launches += 1


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kvad_b200 kernels run on CUDA tensors only; there is no CPU path")


def _rows_view(t: torch.Tensor, what: str) -> int:
    """Leading dimension of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what}: needs a 2-D tensor with contiguous rows, got shape {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0)


class Ops:
    """Kernels bound to one compute dtype."""

    def __init__(self, dtype: torch.dtype):
        self.dtype = dtype
        self.code = _code(dtype)
        self.use_tensor_cores = dtype == torch.bfloat16
        # set to False to keep the bfloat16 engine on the CUDA-core kernels (tests compare both)
        self.tensor_core_linear = dtype == torch.bfloat16 and "linear_tcgen05" in build.sources()
        self.tensor_core_prefill = dtype == torch.bfloat16 and "attention_prefill" in build.sources()
        self.fast_decode = "attention_decode" in build.sources()        # both dtypes: the decode kernel is templated on the storage type
        # Up to 16 rows the product can also run as a stream of weights through registers on the CUDA cores
        # (linear_rows.cu).  Measured on a B200 it beats the tensor-core kernel at one or two rows (qkv at 1 row:
        # 2.4 us against 3.9 us; a GPT-2 small decode step at batch 1: 0.286 ms against 0.326 ms, at batch 2: 0.314
        # against 0.319) and loses from 4 rows on (batch 4: 0.410 ms against 0.327), and it loses on the output head
        # (50257 outputs: the step is 0.307 ms with it, 0.286 without).  So it takes products of at most
        # `rows_linear_max` rows and `ROWS_LINEAR_MAX_OUT` outputs; form="rows" selects it for any count up to 16.
        # In 32-bit there are no tensor cores to lose to: the weight stream is the decode road of the float32 engine
        # for every row count it takes (the tiled CUDA-core kernel would run one row in a tile of 64).
        self._rows_lib = "linear_rows" if dtype == torch.bfloat16 else "linear_rows_f32"     # one library per element type
        self.rows_linear_max = (2 if dtype == torch.bfloat16 else 16) if self._rows_lib in build.sources() else 0
        self.tiled_prompt = True    # prompts that the tensor-core kernel does not take: the tiled CUDA-core kernel, not the row-by-row one
        self._counters = None       # zeroed ints the decode kernel counts finished splits in (left zeroed by it)
        # Two 32-bit buffers [16, width] that q/k/v products of 3..16 rows add their shares of K into (see
        # `linear_sums`); they alternate call by call, and the kernel that reads one clears the other.
        self.qkv_sums = os.environ.get("KVAD_QKV_SUMS", "1") != "0"
        self._sums: Optional[torch.Tensor] = None
        self._sum_calls = 0
        self._sums_open = False         # between a step's first `linear_sums` and its `end_step`
        from . import profile
        if profile.enabled():       # KVAD_PROFILE=1: a table of device time per operation at exit
            profile.instrument(self)

    def path_key(self) -> tuple:
        """Everything on the host that decides which kernels a step of a given shape launches; part of
        the key under which a step's CUDA graph is kept."""
        return (_switch_epoch, self.tensor_core_linear, self.tensor_core_prefill, self.fast_decode,
                self.rows_linear_max, self.qkv_sums, self.SUMS_MIN_K, self.tiled_prompt)

    def begin_step(self) -> None:
        """Called once before a step's first kernel (inside the capture, if the step is being captured)."""
        if self._sums_open and self._sums is not None and not torch.cuda.is_current_stream_capturing():
            self._sums.zero_()              # a step before this one was given up half-way: start clean
        self._sum_calls = 0
        self._sums_open = False

    def end_step(self) -> None:
        """Called once after a step's last kernel.  The two buffers of `linear_sums` alternate and every reader clears
        the one it does not read, so after an even number of such products the first buffer is clean for the next
        step; after an odd number it is cleared here."""
        if self._sum_calls % 2 == 1:
            h = lib("rows")
            _check(h.kvad_zero_bytes(_ptr(self._sums), self._sums[0].numel() * 4, _stream()), h)
        self._sums_open = False

    # -- embedding -----------------------------------------------------------------
    def embed(self, tokens, positions, wte, wpe, out) -> None:
        _need_cuda(tokens, positions, wte, wpe, out)
        n, width = out.shape
        if wte.dtype != self.dtype or (wpe is not None and wpe.dtype != self.dtype):
            raise KernelError(f"embed: tables must be {self.dtype}")
        if out.dtype != torch.float32 or not out.is_contiguous() or wte.shape[1] != width:
            raise KernelError("embed: output must be contiguous float32 of the tables' width")
        if tokens.dtype != torch.int32 or tokens.numel() < n:
            raise KernelError("embed: tokens must be int32, one per row")
        h = lib("rows")
        _check(h.kvad_embed(self.code, _ptr(tokens), _ptr(positions), _ptr(wte), _ptr(wpe), _ptr(out), n, width,
                            wte.shape[0], 0 if wpe is None else wpe.shape[0], _stream()), h)

    # -- norms ---------------------------------------------------------------------
    def layernorm(self, x, gain, bias, eps: float, out, rows=None) -> None:
        _need_cuda(x, gain, bias, out, rows)
        n, width = out.shape
        if x.dtype != torch.float32 or not x.is_contiguous() or x.shape[1] != width:
            raise KernelError("layernorm: input must be the contiguous float32 residual stream")
        if out.dtype != self.dtype or not out.is_contiguous():
            raise KernelError(f"layernorm: output must be contiguous {self.dtype}")
        if gain.numel() != width or (bias is not None and (bias.numel() != width or bias.dtype != gain.dtype)):
            raise KernelError("layernorm: gain and bias must have the row's width and one dtype")
        if rows is None and x.shape[0] < n:
            raise KernelError("layernorm: fewer input rows than output rows")
        if rows is not None and (rows.dtype != torch.int32 or rows.numel() < n):
            raise KernelError("layernorm: row list must be int32, one per output row")
        params_f32 = 1 if gain.dtype == torch.float32 else 0
        if not params_f32 and gain.dtype != torch.bfloat16:
            raise KernelError(f"layernorm: gain must be float32 or bfloat16, not {gain.dtype}")
        h = lib("rows")
        _check(h.kvad_layernorm(self.code, _ptr(x), _ptr(rows), _ptr(gain), _ptr(bias), params_f32, _ptr(out), n, width,
                                float(eps), _stream()), h)

    # -- linear --------------------------------------------------------------------
    ROWS_LINEAR_MAX_OUT = 8192
    ROWS_BLOCKS_MAX = 64           # 32-bit: up to so many rows go through the weight-streaming form in blocks of 16

    def linear(self, a, weight, bias, out, epilogue: str = "store", *, tile: int = 0, splits: int = 0,
               form: str = "auto") -> None:
        """out = epilogue(a . weight^T + bias); weight is [out_features, in_features].

        `form`: "auto"; "rows" (at most 16 rows: weights streamed through registers on the CUDA cores);
        "wide" / "swapped" (the tensor-core kernel's two operand roles).  `tile` and `splits` fix the
        tensor-core kernel's tile width and K split (0: its own choice)."""
        _need_cuda(a, weight, bias, out)
        epi = EPILOGUES[epilogue]
        lda, ldo = _rows_view(a, "linear input"), _rows_view(out, "linear output")
        m, k = a.shape
        n = weight.shape[0]
        if weight.dim() != 2 or weight.shape[1] != k or not weight.is_contiguous():
            raise KernelError(f"linear: weight {tuple(weight.shape)} does not take inputs of width {k}")
        if a.dtype != self.dtype or weight.dtype != self.dtype:
            raise KernelError(f"linear: input and weight must be {self.dtype}")
        want_out = torch.float32 if epi >= 3 else self.dtype
        if out.dtype != want_out or out.shape[0] != m or out.shape[1] != n:
            raise KernelError(f"linear: output must be {want_out} of shape [{m}, {n}]")
        bias_f32 = 0
        if bias is not None:
            if bias.numel() != n:
                raise KernelError(f"linear: bias has {bias.numel()} entries for {n} outputs")
            bias_f32 = 1 if bias.dtype == torch.float32 else 0
            if not bias_f32 and bias.dtype != torch.bfloat16:
                raise KernelError(f"linear: bias must be float32 or bfloat16, not {bias.dtype}")
        ve = 8 if self.dtype == torch.bfloat16 else 4          # elements of a 16-byte piece
        # (beyond ROWS_LINEAR_MAX_OUT outputs - the head - the tensor-core form is as fast or faster, except for one row
        # of long K: 50257 x 1600 at one row 26 us against 44)
        rows_out_ok = self.dtype == torch.float32 or n <= self.ROWS_LINEAR_MAX_OUT or (m == 1 and k >= 1536)
        # (by itself only up to K = 4096: beyond, one column a warp is too long a chain - measured at 1600 x 6400,
        # one row: the tensor-core form with K split over twelve CTAs is 10 % faster on the step)
        # (three and four rows too where the product STORES and K is short - there the tensor-core form needs a cluster:
        # at GPT-2 small's sizes a step of 3 or 4 sequences 0.320 -> 0.301 ms; at K = 1024 and 1600 it loses 1..6 %)
        rows_auto = m <= self.rows_linear_max or (m <= self.rows_linear_max + 2 and epi < 3 and k <= 768 and self.dtype == torch.bfloat16)
        if ((form == "rows" or (form == "auto" and rows_auto and rows_out_ok and k <= 4096)) and m <= 16 and k <= 1024 * ve
                and k % ve == 0 and lda % ve == 0 and (1 << max(0, m - 1).bit_length()) * k * a.element_size() <= 200 * 1024
                and a.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and self._rows_lib in build.sources()):
            h = lib(self._rows_lib)
            _check(h.kvad_linear_rows(self.code, _ptr(a), lda, _ptr(weight), _ptr(bias), bias_f32, _ptr(out), ldo, m, n, k, epi,
                                      _stream()), h)
            return
        if form == "rows":
            raise KernelError("linear: the weight-streaming form takes at most 16 rows and K a multiple of a 16-byte piece, at most 1024 pieces")
        if (form == "auto" and self.dtype == torch.float32 and self.rows_linear_max >= 16 and 16 < m <= self.ROWS_BLOCKS_MAX and k <= 4096
                and k % ve == 0 and lda % ve == 0 and a.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and self._rows_lib in build.sources()):
            # 32-bit, 17..64 rows: the tiled kernel would run a grid of N / 64 CTAs, each walking all of K (17 rows of
            # 768 x 3072: 265 us); the weight-streaming form takes the rows in blocks of up to 16 instead, the later
            # blocks finding the weights in the L2 (a decode step of 17 sequences at GPT-2 small's sizes: 6.1 -> 1.0 ms, of 64: 2.9)
            block = 16
            while block > 1 and block * k * 4 > 200 * 1024:
                block //= 2
            h = lib(self._rows_lib)
            for m0 in range(0, m, block):
                rows = min(block, m - m0)
                _check(h.kvad_linear_rows(self.code, c_void_p(a.data_ptr() + m0 * lda * 4), lda, _ptr(weight), _ptr(bias), bias_f32,
                                          c_void_p(out.data_ptr() + m0 * ldo * 4), ldo, rows, n, k, epi, _stream()), h)
            return
        if self.tensor_core_linear and tcgen05_takes(a, weight, out, lda, ldo):
            h = lib("linear_tcgen05")
            force = (int(tile) & 0xffff) | ((int(splits) & 0xff) << 16) | ({"auto": 0, "wide": 1, "swapped": 2}.get(form, 0) << 24)
            _check(h.kvad_linear_tcgen05(_ptr(a), lda, _ptr(weight), _ptr(bias), bias_f32, _ptr(out), ldo, m, n, k,
                                         epi, force, _stream()), h)
            return
        h = lib("linear_simt")
        _check(h.kvad_linear_simt(self.code, _ptr(a), lda, _ptr(weight), _ptr(bias), bias_f32, _ptr(out), ldo, m, n, k,
                                  epi, _stream()), h)

    SUMS_MIN_K = 1536

    def sums_take(self, m: int, weight, head_dim: int, page_size: int) -> bool:
        """Whether a q/k/v product of `m` rows leaves 32-bit sums for the decode attention to finish (see `linear_sums`).
        Only where K is long (from 1536 on): there the cluster of the storing form costs most (GPT-2 XL's sizes, 8
        rows: +4 % on the step); at K = 768 the two forms are even (+0.8 %) and at K = 1024 this one loses (-1.8 %)."""
        n, k = weight.shape
        return bool(self.qkv_sums and self.dtype == torch.bfloat16 and self.rows_linear_max < m <= 16 and self.tensor_core_linear
                    and self.fast_decode and k % 64 == 0 and k >= self.SUMS_MIN_K and n % 8 == 0 and weight.data_ptr() % 16 == 0 and "linear_tcgen05" in build.sources()
                    and lib("attention_decode").kvad_attention_decode_takes_pre(self.code, int(head_dim), int(page_size)) == 1)

    def linear_sums(self, a, weight):
        """a . weight^T WITHOUT bias as 32-bit sums: the tensor-core product of a few rows splits K over CTAs, and where
        it has to store rounded results the CTAs of a split form a cluster and meet through shared memory; where it
        may ADD, they add their shares atomically and leave - half the time at GPT-2 XL's sizes.  So the product adds into one of two zeroed buffers, and the kernel that reads the sums (the
        decode attention: bias, rounding) clears the other one for the next such product (see `end_step`).  Returns (the sums [rows, outputs], the buffer to clear)."""
        m, n = a.shape[0], weight.shape[0]
        if self._sums is None or self._sums.shape[2] < n:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("linear_sums: its buffers must exist before a step is captured")
            self._sums = torch.zeros((2, 16, (n + 7) // 8 * 8), dtype=torch.float32, device=a.device)
        which = self._sum_calls % 2
        self._sum_calls += 1
        self._sums_open = True
        out = self._sums[which, :m, :n]
        self.linear(a, weight, None, out, "residual")
        return out, self._sums[1 - which]

    def attention_decode_sums(self, sums, bias, k_off: int, v_off: int, clear, out, row_seq, row_pos, page_table, k_pages,
                              v_pages, n_heads: int, scale: float, window: int = 0, *, n_splits: int = 1, scratch=None) -> None:
        """The decode attention with the rows' queries, keys and values given as `linear_sums` left them (queries from
        column 0, keys from `k_off`, values from `v_off`; `bias` as long as a row, or None): the kernel adds the bias,
        rounds, writes the rows' keys and values to the cache, merges its key ranges itself, and clears `clear`."""
        _need_cuda(sums, bias, clear, out, row_seq, row_pos, page_table, k_pages, v_pages, scratch)
        _, n_kv, page, hd = k_pages.shape
        n = sums.shape[0]
        ld_s, ld_o = _rows_view(sums, "q/k/v sums"), _rows_view(out, "attention output")
        if (sums.dtype != torch.float32 or out.dtype != self.dtype or k_pages.dtype != self.dtype or out.shape != (n, n_heads * hd)
                or k_off != n_heads * hd or v_off != k_off + n_kv * hd or sums.shape[1] != v_off + n_kv * hd):
            raise KernelError("attention_decode_sums: sums must be float32 [rows, q | k | v] and match heads x head size")
        bias_f32 = 0
        if bias is not None:
            if bias.numel() != sums.shape[1] or bias.dtype not in (torch.float32, torch.bfloat16):
                raise KernelError("attention_decode_sums: the bias must be as long as a row of sums, float32 or bfloat16")
            bias_f32 = 1 if bias.dtype == torch.float32 else 0
        if n_splits > 1 and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < n * n_heads * n_splits * (hd + 2)):
            raise KernelError("attention_decode_sums: scratch must be float32 with rows x heads x splits x (head_dim + 2) elements")
        counters = None
        if n_splits > 1:
            if self._counters is None or self._counters.numel() < n * n_heads:
                self._counters = torch.zeros(max(4096, n * n_heads), dtype=torch.int32, device=out.device)
            counters = self._counters
        h = lib("attention_decode")
        h.kvad_attention_decode_pre(_ptr(sums), ld_s, _ptr(bias), bias_f32, int(k_off), int(v_off), _ptr(clear),
                                    0 if clear is None else clear.numel())
        _check(h.kvad_attention_decode_step(self.code, c_void_p(0), 0, _ptr(out), ld_o, _ptr(row_seq), _ptr(row_pos),
                                            _ptr(page_table), page_table.shape[1], _ptr(k_pages), _ptr(v_pages),
                                            c_void_p(0), c_void_p(0), 0, _ptr(scratch), _ptr(counters), n, n_heads,
                                            n_kv, hd, page, int(n_splits), float(scale), int(window or 0), _stream()), h)

    # -- cache writes and attention --------------------------------------------------
    def kv_store(self, k_src, v_src, row_seq, row_pos, page_table, k_pages, v_pages) -> None:
        """Writes rows' keys and values to (sequence, position) in one layer's pages
        `[n_pages, n_kv_heads, page_size, head_dim]`."""
        _need_cuda(k_src, v_src, row_seq, row_pos, page_table, k_pages, v_pages)
        ld = _rows_view(k_src, "kv_store keys")
        if _rows_view(v_src, "kv_store values") != ld or k_src.shape != v_src.shape:
            raise KernelError("kv_store: keys and values must be views of one buffer with one row stride")
        _, n_kv, page, hd = k_pages.shape
        if k_src.shape[1] != n_kv * hd or k_pages.shape != v_pages.shape:
            raise KernelError("kv_store: rows do not match the cache's heads")
        if k_src.dtype != self.dtype or k_pages.dtype != self.dtype or not k_pages.is_contiguous() or not v_pages.is_contiguous():
            raise KernelError(f"kv_store: rows and pages must be {self.dtype}, pages contiguous")
        h = lib("rows")
        _check(h.kvad_kv_store(self.code, _ptr(k_src), _ptr(v_src), ld, _ptr(row_seq), _ptr(row_pos), _ptr(page_table),
                               page_table.shape[1], _ptr(k_pages), _ptr(v_pages), k_src.shape[0], n_kv, hd, page,
                               _stream()), h)

    def attention(self, q, out, row_seq, row_pos, page_table, k_pages, v_pages, n_heads: int, scale: float,
                  window: int = 0) -> None:
        """Every row attends over its own sequence's cached keys up to its own position
        (general kernel: any rows, any head size up to 512)."""
        _need_cuda(q, out, row_seq, row_pos, page_table, k_pages, v_pages)
        ld_q, ld_o = _rows_view(q, "attention queries"), _rows_view(out, "attention output")
        _, n_kv, page, hd = k_pages.shape
        if q.shape[1] != n_heads * hd or out.shape[1] != n_heads * hd or q.shape[0] != out.shape[0]:
            raise KernelError("attention: queries/output do not match heads x head size")
        if q.dtype != self.dtype or out.dtype != self.dtype or k_pages.dtype != self.dtype:
            raise KernelError(f"attention: tensors must be {self.dtype}")
        h = lib("attention_simt")
        _check(h.kvad_attention_simt(self.code, _ptr(q), ld_q, _ptr(out), ld_o, _ptr(row_seq), _ptr(row_pos),
                                     _ptr(page_table), page_table.shape[1], _ptr(k_pages), _ptr(v_pages), q.shape[0],
                                     n_heads, n_kv, hd, page, float(scale), int(window or 0), _stream()), h)

    def prompt_takes(self, head_dim: int, page_size: int) -> bool:
        """Whether the tiled CUDA-core kernel for prompts takes this head size and page size."""
        return head_dim % 4 == 0 and head_dim <= 256 and page_size == 64

    def attention_prompt(self, q, out, seq_starts, kv_lens, n_seqs: int, max_new: int, page_table, k_pages, v_pages,
                         n_heads: int, scale: float, window: int = 0) -> None:
        """Rows of sequences packed one after another (`seq_starts`), each sequence's rows being its last positions
        (`kv_lens` is its length after the step): causal attention on the CUDA cores in 32-bit arithmetic, a page of
        keys brought into shared memory once for 32 rows (the float32 engine's prompts; in bfloat16 the head sizes
        the tensor-core kernel refuses)."""
        _need_cuda(q, out, seq_starts, kv_lens, page_table, k_pages, v_pages)
        ld_q, ld_o = _rows_view(q, "attention queries"), _rows_view(out, "attention output")
        _, n_kv, page, hd = k_pages.shape
        if q.shape[1] != n_heads * hd or out.shape[1] != n_heads * hd or q.shape[0] != out.shape[0]:
            raise KernelError("attention_prompt: queries/output do not match heads x head size")
        if q.dtype != self.dtype or out.dtype != self.dtype or k_pages.dtype != self.dtype:
            raise KernelError(f"attention_prompt: tensors must be {self.dtype}")
        h = lib("attention_simt")
        _check(h.kvad_attention_tiled(self.code, _ptr(q), ld_q, _ptr(out), ld_o, _ptr(seq_starts), _ptr(kv_lens), _ptr(page_table),
                                      page_table.shape[1], _ptr(k_pages), _ptr(v_pages), int(n_seqs), n_heads, n_kv, hd, page,
                                      int(max_new), float(scale), int(window or 0), _stream()), h)

    PREFILL_HEAD_SIZES = (16, 32, 48, 64, 80, 96, 112, 128)

    def prefill_takes(self, head_dim: int) -> bool:
        return head_dim in self.PREFILL_HEAD_SIZES

    def prompt_attention_takes(self, q, head_dim: int, page_size: int) -> bool:
        """Whether prompt rows of a mixer other than the plain causal attention (grouped heads, a scale of its own, but
        nothing else on the scores, keys as long as values) go to `attention_prefill`: bfloat16, a head size it has,
        its page size, a positive scale is the caller's; queries on a 16-byte boundary with such a row stride."""
        return (self.tensor_core_prefill and self.prefill_takes(head_dim) and page_size == 64 and q.dtype == torch.bfloat16
                and q.stride(1) == 1 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)

    def attention_prefill(self, q, out, seq_starts, kv_lens, n_seqs: int, max_new: int, page_table, k_pages, v_pages,
                          n_heads: int, scale: float, window: int = 0) -> None:
        """Rows of sequences packed one after another (`seq_starts`), each sequence's rows being its
        last positions (`kv_lens` is its length after the step): causal attention on the tensor cores."""
        _need_cuda(q, out, seq_starts, kv_lens, page_table, k_pages, v_pages)
        ld_q, ld_o = _rows_view(q, "attention queries"), _rows_view(out, "attention output")
        _, n_kv, page, hd = k_pages.shape
        if q.shape[1] != n_heads * hd or out.shape[1] != n_heads * hd or q.shape[0] != out.shape[0]:
            raise KernelError("attention_prefill: queries/output do not match heads x head size")
        if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16:
            raise KernelError("attention_prefill: tensors must be bfloat16")
        h = lib("attention_prefill")
        _check(h.kvad_attention_prefill(_ptr(q), ld_q, q.shape[0], _ptr(out), ld_o, _ptr(seq_starts), _ptr(kv_lens),
                                        _ptr(page_table), page_table.shape[1], _ptr(k_pages), _ptr(v_pages),
                                        k_pages.shape[0], int(n_seqs), n_heads, n_kv, hd, page, int(max_new), float(scale),
                                        int(window or 0), _stream()), h)

    DECODE_HEAD_SIZES = (16, 32, 48, 64, 80, 96, 112, 128, 256)

    def decode_takes(self, head_dim: int) -> bool:
        return head_dim in self.DECODE_HEAD_SIZES

    @staticmethod
    def decode_splits(n_rows: int, n_heads: int, table_width: int, n_sms: Optional[int] = None) -> int:
        """Into how many key ranges a decode step cuts each (row, head): as many as keep the launch one wave
        of CTAs (2.75 an SM; three fit), six at most, one range per page at most.  Measured on a B200 at 12
        heads and ~520 keys, step time in ms by ranges: 4 rows 5: .308, 6: .311, 8: .322; 8 rows 4: .328,
        5: .353; 12 rows 2: .359, 3: .387; 16 rows 1: .394, 2: .366, 3: .405; 24 rows 1: .432, 2: .475.
        Depends on the batch's size only, never on lengths."""
        want = (11 * (n_sms or sm_count())) // (4 * max(1, n_rows * n_heads))
        return max(1, min(want, table_width, 6))          # (the splits of a row and head form one cluster: 8 at most)

    def attention_decode(self, q, out, row_seq, row_pos, page_table, k_pages, v_pages, n_heads: int, scale: float,
                         window: int = 0, *, n_splits: int = 1, scratch=None, k_new=None, v_new=None,
                         merge_in_kernel: bool = False) -> None:
        """Single-token rows over the cache, keys split over CTAs (decode kernel).

        `scratch`: float32, `n_rows * n_heads * n_splits * (head_dim + 2)` elements when `n_splits > 1`.
        `k_new` / `v_new`: this step's keys and values of the rows (views `[rows, kv_heads * head_dim]` of
        one buffer); given, the kernel reads each row's own position from them and writes it to the
        cache itself.  `merge_in_kernel`: the CTA that finishes last merges the splits (else a second kernel)."""
        _need_cuda(q, out, row_seq, row_pos, page_table, k_pages, v_pages, scratch, k_new, v_new)
        ld_q, ld_o = _rows_view(q, "attention queries"), _rows_view(out, "attention output")
        _, n_kv, page, hd = k_pages.shape
        n = q.shape[0]
        if q.shape[1] != n_heads * hd or out.shape[1] != n_heads * hd or out.shape[0] != n:
            raise KernelError("attention_decode: queries/output do not match heads x head size")
        if q.dtype != self.dtype or out.dtype != self.dtype or k_pages.dtype != self.dtype:
            raise KernelError(f"attention_decode: tensors must be {self.dtype}")
        if n_splits > 1 and (scratch is None or scratch.dtype != torch.float32
                             or scratch.numel() < n * n_heads * n_splits * (hd + 2)):
            raise KernelError("attention_decode: scratch must be float32 with rows x heads x splits x (head_dim + 2) elements")
        ld_new = 0
        if k_new is not None:
            ld_new = _rows_view(k_new, "new keys")
            if (v_new is None or _rows_view(v_new, "new values") != ld_new or k_new.shape != (n, n_kv * hd)
                    or v_new.shape != k_new.shape or k_new.dtype != self.dtype or v_new.dtype != self.dtype):
                raise KernelError("attention_decode: new keys and values must be views [rows, kv_heads x head size] of one buffer")
        counters = None
        if merge_in_kernel and n_splits > 1:
            if self._counters is None or self._counters.numel() < n * n_heads:
                self._counters = torch.zeros(max(4096, n * n_heads), dtype=torch.int32, device=q.device)
            counters = self._counters
        h = lib("attention_decode")
        _check(h.kvad_attention_decode_step(self.code, _ptr(q), ld_q, _ptr(out), ld_o, _ptr(row_seq), _ptr(row_pos),
                                            _ptr(page_table), page_table.shape[1], _ptr(k_pages), _ptr(v_pages),
                                            _ptr(k_new), _ptr(v_new), ld_new, _ptr(scratch), _ptr(counters), n, n_heads,
                                            n_kv, hd, page, int(n_splits), float(scale), int(window or 0), _stream()), h)
        if n_splits > 1 and counters is None:
            global _launches
            _launches += 1          # the merge kernel

    # -- RMS norms, rotary positions, gates ---------------------------------------------
    def rmsnorm(self, x, weight, eps: float, out, *, unit_offset: bool = False, rows=None, deferred=None) -> None:
        """out = x / sqrt(mean(x^2) + eps) * w per row (`weight` None: no weight; `unit_offset`: the weight is stored
        around zero and 1 is added).  `x` is the 32-bit residual stream or activations of the compute dtype, and may
        be a view of some columns; `rows`: only these rows of x.  `deferred` = (delta, mult): a scaled sum still owed
        to the stream - the rows are normalised as x + mult * delta; when all rows are walked the sum is written into
        x and delta is cleared."""
        _need_cuda(x, weight, out, rows)
        n, width = out.shape
        ld_in, ld_out = _rows_view(x, "rmsnorm input"), _rows_view(out, "rmsnorm output")
        if (x.shape[1] != width or x.dtype not in (torch.float32, self.dtype)
                or not (out.dtype == self.dtype or (out.dtype == torch.float32 and x.dtype == torch.float32))):
            raise KernelError(f"rmsnorm: input must be float32 or {self.dtype} and as wide as the output ({self.dtype}, or float32 from float32)")
        if rows is None and x.shape[0] < n:
            raise KernelError("rmsnorm: fewer input rows than output rows")
        if rows is not None and (rows.dtype != torch.int32 or rows.numel() < n):
            raise KernelError("rmsnorm: row list must be int32, one per output row")
        w_f32 = 0
        if weight is not None:
            if weight.numel() != width or weight.dtype not in (torch.float32, torch.bfloat16):
                raise KernelError("rmsnorm: the weight must have the row's width, float32 or bfloat16")
            w_f32 = 1 if weight.dtype == torch.float32 else 0
        h = lib("norm_rotary")
        if deferred is not None:
            delta, mult = deferred
            if (x.dtype != torch.float32 or not x.is_contiguous() or delta.dtype != torch.float32 or not delta.is_contiguous()
                    or delta.shape != x.shape):
                raise KernelError("rmsnorm: a deferred sum goes with the contiguous float32 stream and a sum of its shape")
            _check(h.kvad_residual_rmsnorm(_code(out.dtype), _ptr(x), _ptr(delta), float(mult), 1 if rows is None else 0, _ptr(rows),
                                           _ptr(weight), w_f32, int(unit_offset), _ptr(out), ld_out, n, width, float(eps), _stream()), h)
            return
        _check(h.kvad_rmsnorm(_code(x.dtype), _code(out.dtype), _ptr(x), ld_in, _ptr(rows), _ptr(weight), w_f32, int(unit_offset), _ptr(out),
                              ld_out, n, width, float(eps), _stream()), h)

    def scale_add(self, x, delta, mult: float) -> None:
        """x += mult * delta; delta = 0 (both the contiguous float32 stream's shape)."""
        _need_cuda(x, delta)
        if x.dtype != torch.float32 or delta.dtype != torch.float32 or x.shape != delta.shape or not x.is_contiguous() or not delta.is_contiguous():
            raise KernelError("scale_add: needs two contiguous float32 tensors of one shape")
        h = lib("norm_rotary")
        _check(h.kvad_scale_add(_ptr(x), _ptr(delta), float(mult), x.numel(), _stream()), h)

    def zero(self, t) -> None:
        """Clears a contiguous tensor in stream order."""
        _need_cuda(t)
        if not t.is_contiguous():
            raise KernelError("zero: needs a contiguous tensor")
        h = lib("rows")
        _check(h.kvad_zero_bytes(_ptr(t), t.numel() * t.element_size(), _stream()), h)

    def rotary(self, src, dst, row_pos, inv_freq, n_heads: int, dims: int, *, interleaved: bool, head_stride_src: int,
               offset_src: int = 0, head_stride_dst: Optional[int] = None, offset_dst: Optional[int] = None, inverse: bool = False,
               head_gate=None) -> None:
        """Turns the pairs of `dims` entries of each of `n_heads` heads of every row by the row's position times
        `inv_freq[pair]` (32-bit angles): head h's entries start at column h * head_stride + offset.  `dst` may be
        `src` (in place) or another buffer (a copy that turns).  `interleaved`: pairs (2i, 2i+1), else (i, i + dims/2).
        `inverse`: by the negative angle.  `head_gate` [rows, heads]: the turned entries of head h are also multiplied by
        sigmoid(head_gate[r, h])."""
        _need_cuda(src, dst, row_pos, inv_freq, head_gate)
        ld_g = 0
        if head_gate is not None:
            ld_g = _rows_view(head_gate, "rotary head gate")
            if head_gate.dtype != self.dtype or head_gate.shape != (src.shape[0], n_heads):
                raise KernelError("rotary: the head gate must be [rows, heads] of the compute dtype")
            if dims != (head_stride_src if head_stride_dst is None else head_stride_dst):
                raise KernelError("rotary: a head gate goes with heads that are turned whole")
        ld_s, ld_d = _rows_view(src, "rotary input"), _rows_view(dst, "rotary output")
        hs_d = head_stride_src if head_stride_dst is None else head_stride_dst
        off_d = offset_src if offset_dst is None else offset_dst
        n = src.shape[0]
        if (src.dtype != self.dtype or dst.dtype != self.dtype or dst.shape[0] != n or inv_freq.dtype != torch.float32
                or inv_freq.numel() < dims // 2 or row_pos.dtype != torch.int32 or row_pos.numel() < n):
            raise KernelError("rotary: needs rows of the compute dtype, int32 positions and float32 frequencies, one per pair")
        if ((n_heads - 1) * head_stride_src + offset_src + dims > src.shape[1] or (n_heads - 1) * hs_d + off_d + dims > dst.shape[1]):
            raise KernelError("rotary: the heads do not fit the rows")
        h = lib("norm_rotary")
        _check(h.kvad_rotary(self.code, _ptr(src), ld_s, int(head_stride_src), int(offset_src), _ptr(dst), ld_d, int(hs_d), int(off_d),
                             _ptr(row_pos), _ptr(inv_freq), n, int(n_heads), int(dims), int(bool(interleaved)), int(bool(inverse)),
                             _ptr(head_gate), ld_g, _stream()), h)

    def postnorm_rmsnorm(self, x, delta, gain, eps_post: float, out=None, weight=None, eps: float = 0.0, *, unit_offset: bool = False,
                         rows=None, plain_out: bool = False) -> None:
        """x += gain * delta / sqrt(mean(delta^2) + eps_post) per row of the 32-bit stream (`gain`: float32, one per column),
        and, where `out` is given, out = rmsnorm(x) with `weight` and `eps`.  With all rows walked (`rows` None) the sum
        replaces x and delta is cleared; with a row list only `out` is written.  `plain_out`: out = x as it is, in out's
        dtype (no norm, no weight) - for a sublayer that reads the stream itself."""
        _need_cuda(x, delta, gain, out, weight, rows)
        if plain_out:
            if weight is not None or out is None:
                raise KernelError("postnorm_rmsnorm: a plain output has no weight")
            eps = -1.0
        width = x.shape[1]
        if (x.dtype != torch.float32 or delta.dtype != torch.float32 or x.shape != delta.shape or not x.is_contiguous() or not delta.is_contiguous()
                or gain.dtype != torch.float32 or gain.numel() != width):
            raise KernelError("postnorm_rmsnorm: the contiguous float32 stream, a sum of its shape and a float32 gain per column")
        n, ld_out, w_f32, code = x.shape[0], 0, 0, self.code
        if out is not None:
            n, ld_out, code = out.shape[0], _rows_view(out, "postnorm_rmsnorm output"), _code(out.dtype)
            if out.shape[1] != width:
                raise KernelError("postnorm_rmsnorm: the output must be as wide as the stream")
            if weight is not None:
                if weight.numel() != width or weight.dtype not in (torch.float32, torch.bfloat16):
                    raise KernelError("postnorm_rmsnorm: the weight must have the row's width, float32 or bfloat16")
                w_f32 = 1 if weight.dtype == torch.float32 else 0
        elif rows is not None:
            raise KernelError("postnorm_rmsnorm: a row list goes with an output")
        if rows is not None and (rows.dtype != torch.int32 or rows.numel() < n):
            raise KernelError("postnorm_rmsnorm: row list must be int32, one per output row")
        if rows is None and x.shape[0] < n:
            raise KernelError("postnorm_rmsnorm: fewer stream rows than output rows")
        h = lib("norm_rotary")
        _check(h.kvad_postnorm_rmsnorm(code, _ptr(x), _ptr(delta), _ptr(gain), float(eps_post), 1 if rows is None else 0, _ptr(rows),
                                       _ptr(weight), w_f32, int(unit_offset), _ptr(out), ld_out, n, width, float(eps), _stream()), h)

    def head_gate(self, x, gate, n_heads: int) -> None:
        """In place: head h of every row of x times sigmoid(gate[r, h]) (`gate` [rows, heads])."""
        _need_cuda(x, gate)
        ld_x, ld_g = _rows_view(x, "head_gate rows"), _rows_view(gate, "head gate")
        if {x.dtype, gate.dtype} != {self.dtype} or gate.shape != (x.shape[0], n_heads) or x.shape[1] % n_heads:
            raise KernelError(f"head_gate: rows of whole heads and a gate [rows, heads], both {self.dtype}")
        h = lib("norm_rotary")
        _check(h.kvad_head_gate(self.code, _ptr(x), ld_x, _ptr(gate), ld_g, x.shape[0], int(n_heads), x.shape[1] // n_heads, _stream()), h)

    def stream_concat(self, x, x0, out) -> None:
        """out = [x | x0] in the compute dtype (x, x0: float32 [rows, width], contiguous; out [rows, 2 width], contiguous)."""
        _need_cuda(x, x0, out)
        n, width = x.shape
        if (x.dtype != torch.float32 or x0.dtype != torch.float32 or x0.shape != x.shape or not x.is_contiguous() or not x0.is_contiguous()
                or out.dtype != self.dtype or out.shape != (n, 2 * width) or not out.is_contiguous()):
            raise KernelError(f"stream_concat: two contiguous float32 streams of one shape into [rows, 2 width] of {self.dtype}")
        h = lib("norm_rotary")
        _check(h.kvad_stream_concat(self.code, _ptr(x), _ptr(x0), _ptr(out), n, width, _stream()), h)

    def cast_rows(self, x, out, rows=None) -> None:
        """out = x in out's dtype: rows of the contiguous float32 stream (`rows`: an int32 list of them, else the first ones)."""
        _need_cuda(x, out, rows)
        n, width = out.shape
        if x.dtype != torch.float32 or not x.is_contiguous() or x.shape[1] != width or (rows is None and x.shape[0] < n):
            raise KernelError("cast_rows: rows of the contiguous float32 stream, as wide as the output")
        if rows is not None and (rows.dtype != torch.int32 or rows.numel() < n):
            raise KernelError("cast_rows: row list must be int32, one per output row")
        h = lib("norm_rotary")
        _check(h.kvad_cast_rows(_code(out.dtype), _ptr(x), _ptr(rows), _ptr(out), _rows_view(out, "cast_rows output"), n, width, _stream()), h)

    def pair_norm_sum(self, a, b, gain_a, gain_b, delta, eps: float, mult: float = 0.5) -> None:
        """delta += mult * (gain_a * a / rms(a) + gain_b * b / rms(b)) row by row; a = 0; b = 0.  All float32 and contiguous,
        one shape; the gains one number per column."""
        _need_cuda(a, b, gain_a, gain_b, delta)
        n, width = delta.shape
        if (any(t.dtype != torch.float32 or not t.is_contiguous() for t in (a, b, gain_a, gain_b, delta)) or a.shape != delta.shape
                or b.shape != delta.shape or gain_a.numel() != width or gain_b.numel() != width):
            raise KernelError("pair_norm_sum: three contiguous float32 tensors of one shape and two float32 gains per column")
        h = lib("norm_rotary")
        _check(h.kvad_pair_norm_sum(_ptr(a), _ptr(b), _ptr(gain_a), _ptr(gain_b), _ptr(delta), n, width, float(eps), float(mult), _stream()), h)

    def tanh_cap(self, x, cap: float) -> None:
        """x = cap * tanh(x / cap) in place (contiguous float32)."""
        _need_cuda(x)
        if x.dtype != torch.float32 or not x.is_contiguous() or not cap > 0:
            raise KernelError("tanh_cap: a contiguous float32 tensor and a positive cap")
        h = lib("norm_rotary")
        _check(h.kvad_tanh_cap(_ptr(x), x.numel(), float(cap), _stream()), h)

    GATES = {"silu": 0, "sigmoid": 1, "relu": 2, "gelu_tanh": 3}

    def gate_mul(self, gate, value, out, act: str = "silu") -> None:
        """out = act(gate) * value, element by element (`gate`, `value`: views of equal shape, 32-bit arithmetic)."""
        _need_cuda(gate, value, out)
        ld_a, ld_b, ld_o = _rows_view(gate, "gate"), _rows_view(value, "gated values"), _rows_view(out, "gate_mul output")
        if gate.shape != value.shape or out.shape != gate.shape or {gate.dtype, value.dtype, out.dtype} != {self.dtype}:
            raise KernelError(f"gate_mul: needs three {self.dtype} tensors of one shape")
        h = lib("norm_rotary")
        _check(h.kvad_gate_mul(self.code, _ptr(gate), ld_a, _ptr(value), ld_b, _ptr(out), ld_o, gate.shape[0], gate.shape[1],
                               self.GATES[act], _stream()), h)

    # -- attention with shaped scores ---------------------------------------------------
    def kv_store_blend(self, k_src, v_src, row_seq, row_pos, page_table, k_pages, v_pages, *, v_other=None, blend=None) -> None:
        """Rows' keys `[rows, kv heads x dk]` and values `[rows, kv heads x dv]` to their places in the pages
        `[pages, kv heads, 64, dk]` / `[.., dv]`.  With `v_other` (same shape as the values) and `blend` (a scalar in
        device memory) the stored value is (1 - blend) v + blend v_other."""
        _need_cuda(k_src, v_src, row_seq, row_pos, page_table, k_pages, v_pages, v_other, blend)
        ld_k, ld_v = _rows_view(k_src, "keys"), _rows_view(v_src, "values")
        _, n_kv, page, dk = k_pages.shape
        dv = v_pages.shape[3]
        n = k_src.shape[0]
        if (k_src.shape[1] != n_kv * dk or v_src.shape != (n, n_kv * dv) or v_pages.shape[:3] != k_pages.shape[:3]
                or {k_src.dtype, v_src.dtype, k_pages.dtype, v_pages.dtype} != {self.dtype} or not k_pages.is_contiguous() or not v_pages.is_contiguous()):
            raise KernelError(f"kv_store_blend: rows must match the cache's heads and be {self.dtype}")
        ld_o, lam_f32 = 0, 0
        if v_other is not None:
            ld_o = _rows_view(v_other, "the other values")
            if v_other.shape != v_src.shape or v_other.dtype != self.dtype or blend is None or blend.numel() != 1 or blend.dtype not in (torch.float32, torch.bfloat16):
                raise KernelError("kv_store_blend: the other values must have the values' shape, the weight is one float32 or bfloat16 number")
            lam_f32 = 1 if blend.dtype == torch.float32 else 0
        h = lib("attention_scored")
        _check(h.kvad_kv_store_blend(self.code, _ptr(k_src), ld_k, _ptr(v_src), ld_v, _ptr(v_other), ld_o, _ptr(blend if v_other is not None else None),
                                     lam_f32, _ptr(row_seq), _ptr(row_pos), _ptr(page_table), page_table.shape[1], _ptr(k_pages), _ptr(v_pages),
                                     n, n_kv, dk, dv, page, _stream()), h)

    def turn_store(self, q, k_src, v_src, row_seq, row_pos, page_table, k_pages, v_pages, n_heads: int, *, inv_freq=None, dims: int = 0,
                   interleaved: bool = False, value_inv_freq=None, value_interleaved: bool = False) -> None:
        """One pass over a step's rows: the first `dims` entries of every query head turned in place by the row's position
        (pairs (2i, 2i+1) if `interleaved`, else (i, i + dims/2); `inv_freq` one frequency per pair, 32-bit angles), the keys
        turned likewise on their way into the pages, the values turned over ALL their entries (`value_inv_freq` given) or
        stored as they are.  What `rotary` on queries and keys, `rotary` on values and `kv_store_blend` do in three."""
        _need_cuda(q, k_src, v_src, row_seq, row_pos, page_table, k_pages, v_pages, inv_freq, value_inv_freq)
        ld_q, ld_k, ld_v = _rows_view(q, "queries"), _rows_view(k_src, "keys"), _rows_view(v_src, "values")
        _, n_kv, page, dk = k_pages.shape
        dv, n = v_pages.shape[3], q.shape[0]
        if (q.shape[1] != n_heads * dk or k_src.shape != (n, n_kv * dk) or v_src.shape != (n, n_kv * dv) or v_pages.shape[:3] != k_pages.shape[:3]
                or {q.dtype, k_src.dtype, v_src.dtype, k_pages.dtype, v_pages.dtype} != {self.dtype} or not k_pages.is_contiguous()
                or not v_pages.is_contiguous()):
            raise KernelError(f"turn_store: rows must match the cache's heads and be {self.dtype}")
        if dims and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() < dims // 2 or dims % 2 or dims > dk):
            raise KernelError("turn_store: an even number of a key's entries turns, with a float32 frequency per pair")
        if value_inv_freq is not None and (value_inv_freq.dtype != torch.float32 or dv % 2 or value_inv_freq.numel() < dv // 2):
            raise KernelError("turn_store: values turn whole: an even size and a float32 frequency per pair")
        if row_pos.dtype != torch.int32 or row_seq.dtype != torch.int32 or row_pos.numel() < n or row_seq.numel() < n:
            raise KernelError("turn_store: int32 sequences and positions, one per row")
        h = lib("attention_scored")
        _check(h.kvad_turn_store(self.code, _ptr(q), ld_q, _ptr(k_src), ld_k, _ptr(v_src), ld_v, _ptr(inv_freq if dims else None), int(dims),
                                 int(bool(interleaved)), _ptr(value_inv_freq), int(bool(value_interleaved)), _ptr(row_seq), _ptr(row_pos),
                                 _ptr(page_table), page_table.shape[1], _ptr(k_pages), _ptr(v_pages), n, int(n_heads), n_kv, dk, dv, page,
                                 _stream()), h)

    def norm_turn_store(self, q, k_src, v_src, row_seq, row_pos, page_table, k_pages, v_pages, n_heads: int, *, q_weight=None, k_weight=None,
                        span_q: int = 0, span_k: int = 0, eps: float = 0.0, inv_freq=None, dims: int = 0, mscale: float = 1.0) -> None:
        """One pass over a step's rows: queries and keys RMS-normed in 32-bit over `span_q` / `span_k` consecutive entries of
        their projection at a time (a head's size: head by head; the projection's: all heads at once; 0: no norm) with weights
        as long as a span, then the first `dims` entries of every head turned by the row's position (pairs (i, i + dims/2),
        cosine and sine times `mscale`); queries in place, keys on their way into the pages, values stored as they are.  The
        values' pages may have fewer heads than the keys' (several key heads to one value head)."""
        _need_cuda(q, k_src, v_src, row_seq, row_pos, page_table, k_pages, v_pages, q_weight, k_weight, inv_freq)
        ld_q, ld_k, ld_v = _rows_view(q, "queries"), _rows_view(k_src, "keys"), _rows_view(v_src, "values")
        _, n_kv, page, dk = k_pages.shape
        n_v, dv, n = v_pages.shape[1], v_pages.shape[3], q.shape[0]
        if (q.shape[1] != n_heads * dk or k_src.shape != (n, n_kv * dk) or v_src.shape != (n, n_v * dv) or v_pages.shape[0] != k_pages.shape[0]
                or v_pages.shape[2] != page or {q.dtype, k_src.dtype, v_src.dtype, k_pages.dtype, v_pages.dtype} != {self.dtype}
                or not k_pages.is_contiguous() or not v_pages.is_contiguous()):
            raise KernelError(f"norm_turn_store: rows must match the cache's heads and be {self.dtype}")
        if dims and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() < dims // 2 or dims % 2 or dims > dk):
            raise KernelError("norm_turn_store: an even number of a key's entries turns, with a float32 frequency per pair")
        w_f32 = 1
        for w, span in ((q_weight, span_q), (k_weight, span_k)):
            if w is not None:
                if w.dtype not in (torch.float32, torch.bfloat16) or w.numel() != span or not w.is_contiguous():
                    raise KernelError("norm_turn_store: a norm's weight is as long as what is normed together, float32 or bfloat16")
                w_f32 = 1 if w.dtype == torch.float32 else 0
        if q_weight is not None and k_weight is not None and q_weight.dtype != k_weight.dtype:
            raise KernelError("norm_turn_store: the two weights must be of one dtype")
        if row_pos.dtype != torch.int32 or row_seq.dtype != torch.int32 or row_pos.numel() < n or row_seq.numel() < n:
            raise KernelError("norm_turn_store: int32 sequences and positions, one per row")
        h = lib("attention_scored")
        _check(h.kvad_norm_turn_store(self.code, _ptr(q), ld_q, _ptr(k_src), ld_k, _ptr(v_src), ld_v, _ptr(q_weight), _ptr(k_weight), w_f32,
                                      int(span_q), int(span_k), float(eps), _ptr(inv_freq if dims else None), int(dims),
                                      float(mscale), _ptr(row_seq), _ptr(row_pos), _ptr(page_table), page_table.shape[1], _ptr(k_pages),
                                      _ptr(v_pages), n, int(n_heads), n_kv, n_v, dk, dv, page, _stream()), h)

    def scored_merge_diff(self, scratch, n_splits: int, out, n_heads: int, group: int, lam: float, eps: float, gain: float) -> None:
        """The merge of `attention_scored`'s parts (left with `merge=False`, 2 x `n_heads` query heads of single-token rows laid out
        [kv head][map][head of the group]) and `diff_combine` in one launch: out[r, h] = gain * o / sqrt(mean(o^2) + eps),
        o = a1 - lam * a2."""
        _need_cuda(scratch, out)
        n, total = out.shape
        dv = total // n_heads
        if (scratch.dtype != torch.float32 or out.dtype != self.dtype or dv * n_heads != total or n_heads % group
                or scratch.numel() < n * 2 * n_heads * n_splits * (dv + 2)):
            raise KernelError(f"scored_merge_diff: float32 parts of rows x 2 heads x splits x (value size + 2) and an output [rows, heads x dv] of {self.dtype}")
        h = lib("attention_scored")
        _check(h.kvad_scored_merge_diff(self.code, _ptr(scratch), int(n_splits), n, int(n_heads), int(group), dv, _ptr(out),
                                        _rows_view(out, "scored_merge_diff output"), float(lam), float(eps), float(gain), _stream()), h)

    def diff_combine(self, maps, out, n_heads: int, group: int, lam: float, eps: float, gain: float) -> None:
        """out[r, h] = gain * o / sqrt(mean(o^2) + eps), o = a1 - lam * a2 over a head's values, where `maps` (float32
        [rows, 2 heads x dv]) holds the two maps' outputs as [kv head][map][head of the group][dv] and h = kv head x group + head
        of the group."""
        _need_cuda(maps, out)
        n, total = out.shape
        dv = total // n_heads
        if (maps.dtype != torch.float32 or out.dtype != self.dtype or maps.shape != (n, 2 * total) or dv * n_heads != total or n_heads % group):
            raise KernelError(f"diff_combine: float32 maps [rows, 2 heads x dv] and an output [rows, heads x dv] of {self.dtype}")
        h = lib("attention_scored")
        _check(h.kvad_diff_combine(self.code, _ptr(maps), _rows_view(maps, "maps"), _ptr(out), _rows_view(out, "diff_combine output"), n, int(n_heads),
                                   int(group), dv, float(lam), float(eps), float(gain), _stream()), h)

    def latent_store(self, src, weight, eps: float, inv_freq, row_seq, row_pos, page_table, pages, rank: int, rot: int, *,
                     interleaved: bool) -> None:
        """Rows `[rows, rank + rot]`: the first `rank` entries RMS-normalised with `weight`, the last `rot` turned by the
        row's position, stored to pages `[pages, 1, 64, rank + rot]`."""
        _need_cuda(src, weight, inv_freq, row_seq, row_pos, page_table, pages)
        ld = _rows_view(src, "latent rows")
        if (src.shape[1] != rank + rot or pages.shape[1] != 1 or pages.shape[3] != rank + rot or src.dtype != self.dtype or pages.dtype != self.dtype
                or not pages.is_contiguous() or weight.numel() != rank or weight.dtype not in (torch.float32, torch.bfloat16)):
            raise KernelError("latent_store: rows and pages must be [.., rank + rot] of the compute dtype, the weight as long as the rank")
        if rot and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() < rot // 2):
            raise KernelError("latent_store: needs float32 frequencies, one per pair")
        h = lib("attention_scored")
        _check(h.kvad_latent_store(self.code, _ptr(src), ld, _ptr(weight), 1 if weight.dtype == torch.float32 else 0, float(eps), _ptr(inv_freq),
                                   int(bool(interleaved)), _ptr(row_seq), _ptr(row_pos), _ptr(page_table), page_table.shape[1], _ptr(pages),
                                   src.shape[0], int(rank), int(rot), pages.shape[2], _stream()), h)

    HEADS_LINEAR_MAX_ROWS = 64

    def linear_heads(self, a, weight, out, *, head_stride_a: int, head_stride_out: int) -> None:
        """out[r, h * head_stride_out + j] = sum_i weight[h, j, i] * a[r, h * head_stride_a + i] for every head h: one small
        linear map per head (no bias).  Up to `HEADS_LINEAR_MAX_ROWS` rows and 768 inputs a head in ONE launch on the
        CUDA cores (32-bit sums); more rows: one product per head through `linear` (the tensor cores where they take it)."""
        _need_cuda(a, weight, out)
        ld_a, ld_o = _rows_view(a, "head-wise input"), _rows_view(out, "head-wise output")
        if weight.dim() != 3 or not weight.is_contiguous() or {a.dtype, weight.dtype, out.dtype} != {self.dtype} or out.shape[0] != a.shape[0]:
            raise KernelError(f"linear_heads: needs [heads, out, in] weights and rows of {self.dtype}")
        H, n_out, n_in = weight.shape
        if (H - 1) * head_stride_a + n_in > a.shape[1] or (H - 1) * head_stride_out + n_out > out.shape[1]:
            raise KernelError("linear_heads: the heads do not fit the rows")
        n = a.shape[0]
        if n <= self.HEADS_LINEAR_MAX_ROWS and n_in <= 768:
            h = lib("attention_scored")
            _check(h.kvad_linear_heads(self.code, _ptr(a), ld_a, int(head_stride_a), _ptr(weight), _ptr(out), ld_o, int(head_stride_out),
                                       n, H, n_in, n_out, _stream()), h)
            return
        for hd in range(H):
            self.linear(a[:, hd * head_stride_a: hd * head_stride_a + n_in], weight[hd], None,
                        out[:, hd * head_stride_out: hd * head_stride_out + n_out])

    def attention_scored(self, q, out, seq_starts, kv_lens, n_seqs: int, max_new: int, page_table, k_pages, v_pages, n_heads: int,
                         scale: float, *, value_dim: Optional[int] = None, softcap: float = 0.0, slope_span: float = 0.0,
                         window: int = 0, keep_first: int = 0, gate=None, heads_per_block: int = 1, n_splits: int = 1,
                         scratch=None, key_maps: int = 1, merge: bool = True) -> None:
        """Softmax attention of packed rows (each sequence's rows are its last positions) over the paged cache with
        shaped scores: s = q.k * scale, capped by `softcap` * tanh(s / softcap) if positive, less slope_h * distance with
        slope_h = 2^(-slope_span (h+1) / n_heads) if `slope_span` is positive; a row sees the last `window` positions
        (0: all) and always the first `keep_first`.  `v_pages` None: the values are the first `value_dim` entries of the
        keys.  `gate`: the output is multiplied by sigmoid(gate).  `n_splits` > 1 (single-token rows): the keys of a
        row and head are dealt out to that many blocks and merged by a second kernel through `scratch` (float32, rows x
        heads x n_splits x (value size + 2)).  `key_maps` > 1: that many consecutive key heads read one value head (the values'
        pages have kv heads / key_maps heads).  `out` may be float32 whatever the compute dtype (no gate then).  `merge` False (with
        `n_splits` > 1): the parts stay in `scratch` for a merge of the caller's (`scored_merge_diff`), `out` is not written.  32-bit
        arithmetic on the CUDA cores."""
        _need_cuda(q, out, seq_starts, kv_lens, page_table, k_pages, v_pages, gate)
        ld_q, ld_o = _rows_view(q, "attention queries"), _rows_view(out, "attention output")
        _, n_kv, page, dk = k_pages.shape
        if v_pages is None:
            dv, v_ptr = int(value_dim or dk), k_pages
        else:
            dv, v_ptr = v_pages.shape[3], v_pages
            if (v_pages.shape[0] != k_pages.shape[0] or v_pages.shape[1] * key_maps != n_kv or v_pages.shape[2] != page
                    or v_pages.dtype != self.dtype or not v_pages.is_contiguous()):
                raise KernelError("attention_scored: the values' pages must match the keys'")
        if q.shape[1] != n_heads * dk or out.shape != (q.shape[0], n_heads * dv):
            raise KernelError("attention_scored: queries/output do not match heads x sizes")
        if {q.dtype, k_pages.dtype} != {self.dtype} or out.dtype not in (self.dtype, torch.float32) or not k_pages.is_contiguous():
            raise KernelError(f"attention_scored: tensors must be {self.dtype}")
        out_f32 = out.dtype == torch.float32 and self.dtype != torch.float32
        if out_f32 and gate is not None:
            raise KernelError("attention_scored: a float32 output takes no gate")
        ld_g = 0
        if gate is not None:
            ld_g = _rows_view(gate, "attention gate")
            if gate.shape != out.shape or gate.dtype != self.dtype:
                raise KernelError("attention_scored: the gate must have the output's shape and dtype")
        if n_splits > 1 and (max_new != 1 or scratch is None or scratch.dtype != torch.float32
                             or scratch.numel() < q.shape[0] * n_heads * n_splits * (dv + 2)):
            raise KernelError("attention_scored: splitting keys goes with single-token rows and float32 scratch of rows x heads x splits x (value size + 2)")
        h = lib("attention_scored")
        _check(h.kvad_attention_scored(self.code, _ptr(q), ld_q, _ptr(out), ld_o, _ptr(gate), ld_g, _ptr(seq_starts), _ptr(kv_lens),
                                       _ptr(page_table), page_table.shape[1], _ptr(k_pages), _ptr(v_ptr), int(n_seqs), int(n_heads), n_kv,
                                       dk, dv, page, int(max_new), int(heads_per_block), float(scale), float(softcap or 0.0),
                                       float(slope_span or 0.0), int(window or 0), int(keep_first or 0), int(n_splits),
                                       _ptr(scratch if n_splits > 1 else None), int(key_maps), int(out_f32), int(bool(merge)), _stream()), h)
        if n_splits > 1 and merge:
            global _launches
            _launches += 1          # the merge kernel

    @staticmethod
    def scored_splits(n_rows: int, n_kv_heads: int, group: int, reach: int, n_sms: Optional[int] = None, per_sm: int = 2) -> int:
        """Into how many parts single-token rows cut the keys of a (row, key/value head): enough blocks for two
        an SM (`per_sm`), one part per 64 keys of `reach` (the window plus the kept first positions, or the longest sequence the
        cache holds) at most, 16 at most.  Depends on the batch's size and the layer's constants only."""
        blocks = max(1, n_rows * n_kv_heads * -(-group // 32))
        want = (int(per_sm) * (n_sms or sm_count())) // blocks
        return max(1, min(want, -(-reach // 64) + 1, 16))

    # -- retention ------------------------------------------------------------------------
    def retention(self, q, k, v, out, state, seq_starts, kv_lens, seq_slots, n_seqs: int, decay, n_heads: int, *, inv_freq=None,
                  rot_dims: int = 0, interleaved: bool = False, k_scale: float = 1.0, gate=None, unit_norm_eps: Optional[float] = None,
                  raw=None, silu_inputs: bool = False, raw_only: bool = False) -> None:
        """Per sequence and head, over the step's rows in order: S = decay_h S + k v^T, o = S^T q, with q and k turned by
        position first (`inv_freq`, `rot_dims`), k scaled by `k_scale`; `unit_norm_eps`: o over its root mean square per
        head; `gate`: times silu(gate).  `state` is `[slots, heads, dk, dv]` float32 and is carried on.  `raw`: float32
        scratch `[rows, heads x dv]`, needed where `retention_needs_raw` says so (a head's columns spread over blocks).
        `silu_inputs`: q, k and v pass a silu first (32-bit).  `raw_only`: the 32-bit read-outs in `raw` are all that is
        written (`out` may be None; no norm, no gate)."""
        _need_cuda(q, k, v, out, state, seq_starts, kv_lens, seq_slots, decay, inv_freq, gate)
        if raw_only:
            if raw is None or gate is not None or unit_norm_eps is not None:
                raise KernelError("retention: raw read-outs go to `raw`, without norm or gate")
            out = q.new_empty((q.shape[0], 0)) if out is None else out
        ld_q, ld_k, ld_v = (_rows_view(t, "retention rows") for t in (q, k, v))
        ld_o = 0 if raw_only else _rows_view(out, "retention rows")
        if state.dim() != 4 or state.dtype != torch.float32 or not state.is_contiguous() or state.shape[1] != n_heads:
            raise KernelError("retention: the state must be contiguous float32 [slots, heads, dk, dv]")
        dk, dv = state.shape[2], state.shape[3]
        n = q.shape[0]
        if (q.shape[1] != n_heads * dk or k.shape != q.shape or v.shape != (n, n_heads * dv) or (not raw_only and out.shape != v.shape)
                or {q.dtype, k.dtype, v.dtype, out.dtype} != {self.dtype}):
            raise KernelError(f"retention: rows must be {self.dtype} and match heads x sizes of the state")
        if decay.dtype != torch.float32 or decay.numel() != n_heads:
            raise KernelError("retention: one float32 decay per head")
        if rot_dims and (inv_freq is None or inv_freq.dtype != torch.float32 or inv_freq.numel() < rot_dims // 2):
            raise KernelError("retention: needs float32 frequencies, one per pair")
        ld_g = 0
        if gate is not None:
            ld_g = _rows_view(gate, "retention gate")
            if gate.shape != out.shape or gate.dtype != self.dtype:
                raise KernelError("retention: the gate must have the output's shape and dtype")
        if raw is not None and (raw.dtype != torch.float32 or not raw.is_contiguous() or raw.numel() < n * n_heads * dv):
            raise KernelError("retention: the scratch must be contiguous float32 [rows, heads x dv]")
        h = lib("retention")
        _check(h.kvad_retention(self.code, _ptr(q), ld_q, _ptr(k), ld_k, _ptr(v), ld_v, _ptr(gate), ld_g, _ptr(out), ld_o, _ptr(raw), n, _ptr(state),
                                _ptr(seq_starts), _ptr(kv_lens), _ptr(seq_slots), _ptr(decay), _ptr(inv_freq), int(rot_dims),
                                int(bool(interleaved)), int(n_seqs), int(n_heads), dk, dv, float(k_scale),
                                float(unit_norm_eps or 0.0), 0 if unit_norm_eps is None else 1, int(bool(silu_inputs)), 0 if raw_only else 1,
                                _stream()), h)

    def row_norm_gate(self, raw, gate, weight, out, eps: float) -> None:
        """out = raw / sqrt(mean over the row (raw^2) + eps) * weight * sigmoid(gate): `raw` float32, `gate` (may be None) and
        `out` of the compute dtype, `weight` one per column (may be None)."""
        _need_cuda(raw, gate, weight, out)
        n, width = raw.shape
        if raw.dtype != torch.float32 or out.dtype != self.dtype or out.shape != raw.shape:
            raise KernelError(f"row_norm_gate: float32 input and {self.dtype} output of one shape")
        ld_g = 0
        if gate is not None:
            ld_g = _rows_view(gate, "gate")
            if gate.shape != raw.shape or gate.dtype != self.dtype:
                raise KernelError("row_norm_gate: the gate must have the output's shape and dtype")
        w_f32 = 0
        if weight is not None:
            if weight.numel() != width or weight.dtype not in (torch.float32, torch.bfloat16):
                raise KernelError("row_norm_gate: the weight must have the row's width, float32 or bfloat16")
            w_f32 = 1 if weight.dtype == torch.float32 else 0
        h = lib("retention")
        _check(h.kvad_row_norm_gate(self.code, _ptr(raw), _rows_view(raw, "read-outs"), _ptr(gate), ld_g, _ptr(weight), w_f32, _ptr(out),
                                    _rows_view(out, "row_norm_gate output"), n, width, float(eps), _stream()), h)

    def retention_needs_raw(self, dk: int, dv: int) -> bool:
        return lib("retention").kvad_retention_needs_raw(int(dk), int(dv)) == 1

    # -- recurrences with gates that depend on the token ------------------------------------
    RECURRENCES = {"matrix_memory": 0, "delta_rule": 1}

    def recurrence_state_size(self, kind: str, n_heads: int, dk: int, dv: int) -> int:
        """32-bit numbers of state a sequence keeps for one such layer (the matrices in the kernel's own layout, and for
        the matrix memory its normaliser and running maximum)."""
        return int(lib("gated_recurrence").kvad_gated_recurrence_state(self.RECURRENCES[kind], int(n_heads), int(dk), int(dv)))

    def gated_recurrence(self, kind: str, q, k, v, gates, out, state, seq_starts, seq_slots, n_seqs: int, n_heads: int, n_kv_heads: int,
                         dk: int, dv: int, *, q_scale: float = 1.0, cap: float = 0.0, beta=None, a_log=None, dt_bias=None,
                         gates_ready: bool = False) -> None:
        """Per sequence and head over the step's rows in order; `state` is `[slots, floats]` (32-bit), carried on.
        `matrix_memory`: S = exp(f + m' - m) S + exp(i - m) k v^T with the running maximum m, n likewise with k alone,
        o = S^T q / (max(|n.q|, exp(-m)) + 1e-6); `gates` float32 [rows, 2 heads] = raw input | forget projections, capped
        here (`cap` tanh(x / cap)), the forget gate through logsigmoid.  `delta_rule`: S = g * S per key channel,
        u = beta (v - S^T k), S += k u^T, o = S^T q; `gates` float32 [rows, heads x dk] raw, g = exp(-exp(a_log) softplus(gates +
        dt_bias)), or with `gates_ready` g itself (`decay_gate`); `beta` float32 [rows, heads].  q and k have `n_kv_heads` heads that the heads share in groups; `out` is
        float32 [rows, heads x dv], the raw read-out."""
        _need_cuda(q, k, v, gates, out, state, seq_starts, seq_slots, beta, a_log, dt_bias)
        mode = self.RECURRENCES[kind]
        ld_q, ld_k, ld_v, ld_g, ld_o = (_rows_view(t, "recurrence rows") for t in (q, k, v, gates, out))
        n = q.shape[0]
        if (q.shape[1] != n_kv_heads * dk or k.shape != q.shape or v.shape != (n, n_heads * dv) or out.shape != (n, n_heads * dv)
                or len({q.dtype, k.dtype, v.dtype}) != 1 or q.dtype not in (torch.float32, self.dtype)):
            raise KernelError(f"gated_recurrence: q, k, v must be float32 or {self.dtype} and match heads x sizes")
        if gates.dtype != torch.float32 or out.dtype != torch.float32 or gates.shape != (n, 2 * n_heads if mode == 0 else n_heads * dk):
            raise KernelError("gated_recurrence: gates and output must be float32 of the kind's shape")
        if state.dim() != 2 or state.dtype != torch.float32 or not state.is_contiguous() or state.shape[1] < self.recurrence_state_size(kind, n_heads, dk, dv):
            raise KernelError("gated_recurrence: the state must be contiguous float32 [slots, floats] of the layer's size")
        ld_b, p_f32 = 0, 0
        if mode == 1:
            if beta is None or beta.dtype != torch.float32 or beta.shape != (n, n_heads) or a_log is None or dt_bias is None:
                raise KernelError("gated_recurrence: the delta rule needs float32 beta [rows, heads], A_log and dt_bias")
            ld_b = _rows_view(beta, "beta")
            if a_log.numel() != n_heads or dt_bias.numel() != n_heads * dk or a_log.dtype != dt_bias.dtype or a_log.dtype not in (torch.float32, torch.bfloat16):
                raise KernelError("gated_recurrence: A_log per head and dt_bias per head and key channel, one dtype")
            p_f32 = 1 if a_log.dtype == torch.float32 else 0
        h = lib("gated_recurrence")
        _check(h.kvad_gated_recurrence(mode, _code(q.dtype), _ptr(q), ld_q, _ptr(k), ld_k, _ptr(v), ld_v, _ptr(gates), ld_g, _ptr(beta), ld_b,
                                       _ptr(a_log), _ptr(dt_bias), p_f32, _ptr(out), ld_o, _ptr(state), state.stride(0), _ptr(seq_starts),
                                       _ptr(seq_slots), int(n_seqs), int(n_heads), int(n_kv_heads), int(dk), int(dv), float(q_scale),
                                       float(cap), int(bool(gates_ready)), _stream()), h)

    def decay_gate(self, a, a_log, dt_bias, n_heads: int, dk: int) -> None:
        """In place on float32 `a` [rows, heads x dk]: g = exp(-exp(a_log_h) softplus(a + dt_bias))."""
        _need_cuda(a, a_log, dt_bias)
        if (a.dtype != torch.float32 or a.shape[1] != n_heads * dk or a_log.numel() != n_heads or dt_bias.numel() != n_heads * dk
                or a_log.dtype != dt_bias.dtype or a_log.dtype not in (torch.float32, torch.bfloat16)):
            raise KernelError("decay_gate: float32 rows [rows, heads x dk], A_log per head and dt_bias per head and key channel of one dtype")
        h = lib("gated_recurrence")
        _check(h.kvad_decay_gate(_ptr(a), _rows_view(a, "decay rows"), _ptr(a_log), _ptr(dt_bias), 1 if a_log.dtype == torch.float32 else 0,
                                 a.shape[0], int(n_heads), int(dk), _stream()), h)

    def short_conv(self, x, taps, y, state, conv_off: int, row_seq, row_pos, seq_starts, seq_slots, *, n_sigmoid: int = 0,
                   unit_heads: int = 0, unit_dim: int = 0, scaled_heads: int = 0, head_scale: float = 1.0, unit_eps: float = 0.0) -> None:
        """y[:, :C] = silu(causal convolution over time per channel of x[:, :C]) with `taps` [C, n]: the last column meets the
        row itself, inputs before the step's rows come from the sequence's kept inputs (`state[slot, conv_off:]` as
        [n - 1, C]), zeros before position 0.  The first `unit_heads` x `unit_dim` channels are then made unit vectors per head
        (sum of squares + `unit_eps` under the root), the first `scaled_heads` of them times `head_scale`.  The `n_sigmoid`
        columns after the channels are y = sigmoid(x).  y is float32."""
        _need_cuda(x, taps, y, state, row_seq, row_pos, seq_starts, seq_slots)
        ld_x, ld_y = _rows_view(x, "short_conv input"), _rows_view(y, "short_conv output")
        C, n_taps = taps.shape
        n = y.shape[0]
        if (x.dtype != self.dtype or taps.dtype != self.dtype or not taps.is_contiguous() or y.dtype != torch.float32 or x.shape[0] != n
                or x.shape[1] < C + n_sigmoid or y.shape[1] < C + n_sigmoid or state.dtype != torch.float32 or state.dim() != 2
                or state.shape[1] < conv_off + (n_taps - 1) * C):
            raise KernelError(f"short_conv: needs {self.dtype} rows and taps, float32 output and state of matching sizes")
        h = lib("gated_recurrence")
        _check(h.kvad_short_conv(self.code, _ptr(x), ld_x, _ptr(taps), _ptr(y), ld_y, _ptr(state), state.stride(0), int(conv_off),
                                 _ptr(row_seq), _ptr(row_pos), _ptr(seq_starts), _ptr(seq_slots), n, C, n_taps, int(n_sigmoid),
                                 int(unit_heads), int(unit_dim), int(scaled_heads), float(head_scale), float(unit_eps), _stream()), h)

    def conv_state(self, x, n_channels: int, n_taps: int, state, conv_off: int, seq_starts, seq_slots, n_seqs: int) -> None:
        """Keeps every sequence's last `n_taps` - 1 rows of x[:, :n_channels] (older ones from what was kept) for the next step."""
        _need_cuda(x, state, seq_starts, seq_slots)
        ld_x = _rows_view(x, "conv_state input")
        if x.dtype != self.dtype or x.shape[1] < n_channels or state.dtype != torch.float32 or state.shape[1] < conv_off + (n_taps - 1) * n_channels:
            raise KernelError("conv_state: rows of the compute dtype and a float32 state with room for the kept inputs")
        h = lib("gated_recurrence")
        _check(h.kvad_conv_state(self.code, _ptr(x), ld_x, _ptr(state), state.stride(0), int(conv_off), _ptr(seq_starts), _ptr(seq_slots),
                                 int(n_seqs), int(n_channels), int(n_taps), _stream()), h)

    def head_norm_gate(self, raw, gate, weight, out, n_heads: int, eps: float, *, weight_per_head: bool) -> None:
        """out = raw / sqrt(mean over the head (raw^2) + eps) * weight * sigmoid(gate), head by head; `weight` is as long as
        all heads (`weight_per_head`) or as one head; `raw` float32, `gate` and `out` of the compute dtype."""
        _need_cuda(raw, gate, weight, out)
        ld_r, ld_o = _rows_view(raw, "read-out"), _rows_view(out, "normed read-out")
        n, total = raw.shape
        dv = total // n_heads
        if raw.dtype != torch.float32 or out.dtype != self.dtype or out.shape != raw.shape or dv * n_heads != total:
            raise KernelError(f"head_norm_gate: float32 input and {self.dtype} output of one shape, whole heads")
        ld_g = 0
        if gate is not None:
            ld_g = _rows_view(gate, "gate")
            if gate.shape != raw.shape or gate.dtype != self.dtype:
                raise KernelError("head_norm_gate: the gate must have the output's shape and dtype")
        w_f32 = 0
        if weight is not None:
            if weight.numel() != (total if weight_per_head else dv) or weight.dtype not in (torch.float32, torch.bfloat16):
                raise KernelError("head_norm_gate: the weight must be as long as all heads or as one, float32 or bfloat16")
            w_f32 = 1 if weight.dtype == torch.float32 else 0
        h = lib("gated_recurrence")
        _check(h.kvad_head_norm_gate(self.code, _ptr(raw), ld_r, _ptr(gate), ld_g, _ptr(weight), w_f32, int(bool(weight_per_head)), _ptr(out),
                                     ld_o, n, int(n_heads), dv, float(eps), _stream()), h)

    # -- routed feed-forward ------------------------------------------------------------------
    MOE_WIDE_TILE = 128
    MOE_WIDE_MIN_SLOTS = 512

    def moe_tile_rows(self, n_rows: int = 0, top: int = 1, pieces: bool = False) -> int:
        """Positions a tile of the grouped products holds for a step of `n_rows` rows: 128 where the tensor-core form
        runs (bfloat16, from 512 (row, choice) pairs on, `pieces`: both products' input sizes are whole 16-byte pieces),
        else the CUDA-core form's 32.  Depends on the step's shape only."""
        wide = (self.tensor_core_linear and n_rows * top >= self.MOE_WIDE_MIN_SLOTS and pieces)
        return self.MOE_WIDE_TILE if wide else int(lib("moe").kvad_moe_tile_rows())

    @staticmethod
    def moe_max_tiles(n_rows: int, top: int, n_experts: int, tile_rows: int) -> int:
        """How many tiles of positions a step of this shape can need at most, whatever the routing."""
        slots = n_rows * top
        return min(slots, slots // tile_rows + n_experts)

    def moe_route(self, logits, top: int, chosen, weight) -> None:
        """Per row of float32 `logits` [rows, experts]: the `top` largest (ties: the lower index) into int32 `chosen`
        [rows, top], softmax over the chosen logits into float32 `weight` [rows, top]."""
        _need_cuda(logits, chosen, weight)
        n, E = logits.shape
        if (logits.dtype != torch.float32 or chosen.dtype != torch.int32 or weight.dtype != torch.float32 or chosen.shape != (n, top)
                or weight.shape != (n, top) or not chosen.is_contiguous() or not weight.is_contiguous()):
            raise KernelError("moe_route: float32 logits, int32 choices and float32 weights [rows, top]")
        h = lib("moe")
        _check(h.kvad_moe_route(_ptr(logits), _rows_view(logits, "router logits"), n, E, int(top), _ptr(chosen), _ptr(weight), _stream()), h)

    ROUTINGS = {"top_logits": 0, "scores": 1, "sigmoid": 2}

    def moe_sort(self, chosen, n_experts: int, tile_rows: int, tile_expert, pos_row, pos_slot, slot_pos, *, logits=None, weight=None,
                 routing: str = "top_logits", correction=None, n_real: Optional[int] = None) -> None:
        """Groups the (row, choice) slots of `chosen` [rows, top] by expert, every expert's list padded to whole tiles of
        `tile_rows` positions: `tile_expert` [tiles] (-1: unused), `pos_row` / `pos_slot` [tiles x tile_rows] (-1: padding),
        `slot_pos` [rows x top]: where each slot went.  With `logits` and `weight` the same launch routes the rows first
        (as `moe_route` does) and writes `chosen` and `weight`.  `routing` "scores": the scores are the softmax over all
        experts, the `top` largest of score + `correction` (float32, one per expert, or None) are chosen and weigh their
        scores over the chosen scores' sum.  `routing` "sigmoid": the `top` largest logits are chosen and each weighs in with the
        sigmoid of its own logit, not renormalised.  `n_real` < `n_experts`: the experts from `n_real` on have no matrices; their
        slots get no position (`slot_pos` -1)."""
        _need_cuda(chosen, tile_expert, pos_row, pos_slot, slot_pos, logits, weight, correction)
        if correction is not None and (correction.dtype != torch.float32 or correction.numel() != n_experts):
            raise KernelError("moe_sort: the correction is float32, one per expert")
        ld_z = 0
        if logits is not None:
            ld_z = _rows_view(logits, "router logits")
            if (logits.dtype != torch.float32 or logits.shape != (chosen.shape[0], n_experts) or weight is None or weight.dtype != torch.float32
                    or weight.shape != chosen.shape or not weight.is_contiguous()):
                raise KernelError("moe_sort: routing needs float32 logits [rows, experts] and weights [rows, top]")
        n, top = chosen.shape
        tiles = tile_expert.numel()
        if any(t.dtype != torch.int32 or not t.is_contiguous() for t in (chosen, tile_expert, pos_row, pos_slot, slot_pos)) or \
                pos_row.numel() < tiles * tile_rows or pos_slot.numel() < tiles * tile_rows or slot_pos.numel() < n * top:
            raise KernelError("moe_sort: int32 lists, a tile's rows per tile, a place per slot")
        h = lib("moe")
        _check(h.kvad_moe_sort(_ptr(chosen), n * top, top, int(n_experts), tiles, int(tile_rows), _ptr(tile_expert), _ptr(pos_row), _ptr(pos_slot),
                               _ptr(slot_pos), _ptr(logits), ld_z, _ptr(weight), self.ROUTINGS[routing], _ptr(correction),
                               int(n_experts if n_real is None else n_real), _stream()), h)
        if logits is not None and n >= h.kvad_moe_route_apart_rows():
            global _launches
            _launches += 1          # many rows: the routing is a launch of its own

    def gather_rows(self, a, pos_row, out) -> None:
        """out[p] = a[pos_row[p]], zeros where pos_row[p] < 0."""
        _need_cuda(a, pos_row, out)
        ld_a, ld_o = _rows_view(a, "gather input"), _rows_view(out, "gather output")
        if a.dtype != out.dtype or a.shape[1] != out.shape[1] or pos_row.dtype != torch.int32 or pos_row.numel() < out.shape[0]:
            raise KernelError("gather_rows: rows of one dtype and width, an int32 row per output row")
        h = lib("moe")
        _check(h.kvad_gather_rows(_code(a.dtype), _ptr(a), ld_a, _ptr(pos_row), _ptr(out), ld_o, out.shape[0], out.shape[1], _stream()), h)

    MOE_FEW_SLOTS = 128

    def grouped_linear(self, a, weight, out, tile_expert, valid, *, in_rows=None, out_rows=None, few_rows: bool = False) -> None:
        """For every tile t of positions and position p in it: out[out_rows[p]] = weight[tile_expert[t]] . a[in_rows[p]]
        (`weight` [experts, outputs, inputs]; a row list that is None is the position itself; `valid[p]` < 0: padding).
        `out` is of the compute dtype or float32.  Tiles of 128 positions with no row lists run on the tensor cores
        (whole tiles, padding included: the rows of `a` at padding must be finite), tiles of 32 on the CUDA cores: as tiled
        products, or with `few_rows` (a step of at most `MOE_FEW_SLOTS` (row, choice) pairs: most of a tile is padding) as a
        stream of the chosen experts' weights."""
        _need_cuda(a, weight, out, tile_expert, valid, in_rows, out_rows)
        ld_a, ld_o = _rows_view(a, "grouped input"), _rows_view(out, "grouped output")
        if weight.dim() != 3 or not weight.is_contiguous() or a.dtype != self.dtype or weight.dtype != self.dtype or out.dtype not in (self.dtype, torch.float32):
            raise KernelError(f"grouped_linear: needs [experts, out, in] weights and rows of {self.dtype}")
        E, n_out, k = weight.shape
        if a.shape[1] != k or out.shape[1] != n_out:
            raise KernelError("grouped_linear: rows do not match the experts' sizes")
        tiles = tile_expert.numel()
        tile_rows = valid.numel() // max(tiles, 1)
        if tile_rows == self.MOE_WIDE_TILE:
            if in_rows is not None or out_rows is not None or not self.tensor_core_linear or a.shape[0] != tiles * tile_rows or out.shape[0] != a.shape[0]:
                raise KernelError("grouped_linear: tiles of 128 positions run on the tensor cores, rows in position order on both sides")
            h = lib("linear_tcgen05")
            _check(h.kvad_linear_tcgen05_grouped(_ptr(a), ld_a, _ptr(weight), E, _ptr(out), ld_o, _ptr(tile_expert), a.shape[0], n_out, k,
                                                 1 if out.dtype == torch.float32 else 0, _stream()), h)
            return
        h = lib("moe")
        _check(h.kvad_grouped_linear(self.code, 1 if out.dtype == torch.float32 else 0, _ptr(a), ld_a, _ptr(in_rows), _ptr(weight),
                                     weight.stride(0), _ptr(out), ld_o, _ptr(out_rows), _ptr(valid), _ptr(tile_expert), tiles,
                                     n_out, k, int(bool(few_rows)), _stream()), h)

    def clamped_glu(self, gate, up, out, limit: float, alpha: float = 1.702) -> None:
        """out = g sigmoid(alpha g) (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit), 32-bit arithmetic."""
        _need_cuda(gate, up, out)
        ld_g, ld_u, ld_o = _rows_view(gate, "gate"), _rows_view(up, "up"), _rows_view(out, "clamped_glu output")
        if gate.shape != up.shape or out.shape != gate.shape or {gate.dtype, up.dtype, out.dtype} != {self.dtype}:
            raise KernelError(f"clamped_glu: needs three {self.dtype} tensors of one shape")
        h = lib("moe")
        _check(h.kvad_clamped_glu(self.code, _ptr(gate), ld_g, _ptr(up), ld_u, _ptr(out), ld_o, gate.shape[0], gate.shape[1], float(limit),
                                  float(alpha), _stream()), h)

    def scaled_glu(self, gate, up, out, act: str = "silu", slot=None, scale=None) -> None:
        """out = act(s g) * (s u) with s = scale[slot[p]] for row p (`slot` int32 per row, -1: padding, whose output is zero;
        `scale` float32 per (row, choice) pair; both None: s = 1): a gated expert whose INPUT is scaled by the router's weight,
        W (s h) = s (W h).  act: silu or gelu_tanh; 32-bit arithmetic."""
        _need_cuda(gate, up, out, slot, scale)
        ld_g, ld_u, ld_o = _rows_view(gate, "gate"), _rows_view(up, "up"), _rows_view(out, "scaled_glu output")
        if gate.shape != up.shape or out.shape != gate.shape or {gate.dtype, up.dtype, out.dtype} != {self.dtype}:
            raise KernelError(f"scaled_glu: needs three {self.dtype} tensors of one shape")
        if (slot is None) != (scale is None) or (slot is not None and (slot.dtype != torch.int32 or slot.numel() < gate.shape[0]
                                                                        or scale.dtype != torch.float32 or not scale.is_contiguous())):
            raise KernelError("scaled_glu: an int32 pair per row and a float32 scale per pair, or neither")
        h = lib("moe")
        _check(h.kvad_scaled_glu(self.code, _ptr(gate), ld_g, _ptr(up), ld_u, _ptr(out), ld_o, _ptr(slot), _ptr(scale), gate.shape[0], gate.shape[1],
                                 self.GATES[act], _stream()), h)

    def moe_combine(self, residual, outs, slot_pos, weight, identity_input=None, top: Optional[int] = None) -> None:
        """residual[r] += sum_k weight[r, k] * outs[slot_pos[r * top + k]], the choices in order (all float32); a slot
        without a position (-1: an expert whose output is its input) adds weight[r, k] * identity_input[r].  `weight` None
        (then `top` says how many choices a row has): every weight is 1."""
        _need_cuda(residual, outs, slot_pos, weight, identity_input)
        ld_in, in_code = 0, F32
        if identity_input is not None:
            ld_in, in_code = _rows_view(identity_input, "the experts' input"), _code(identity_input.dtype)
            if identity_input.shape != residual.shape:
                raise KernelError("moe_combine: the experts' input must have the stream's shape")
        n, width = residual.shape
        top = weight.shape[1] if weight is not None else int(top)
        if (any(t.dtype != torch.float32 for t in (residual, outs) + (() if weight is None else (weight,))) or not residual.is_contiguous()
                or (weight is not None and (not weight.is_contiguous() or weight.shape[0] != n)) or outs.shape[1] != width or slot_pos.dtype != torch.int32 or slot_pos.numel() < n * top):
            raise KernelError("moe_combine: float32 stream [rows, width], expert outputs [positions, width], weights [rows, top], int32 places")
        h = lib("moe")
        _check(h.kvad_moe_combine(_ptr(residual), _ptr(outs), _rows_view(outs, "expert outputs"), _ptr(slot_pos), _ptr(weight), n, width, top,
                                  in_code, _ptr(identity_input), ld_in, _stream()), h)

    def relu_squared(self, x, out, row_gate=None) -> None:
        """out = max(x, 0)^2, times sigmoid(row_gate[r]) where `row_gate` [rows, 1] is given (32-bit arithmetic)."""
        _need_cuda(x, out, row_gate)
        ld_x, ld_o, ld_g = _rows_view(x, "relu_squared input"), _rows_view(out, "relu_squared output"), 0
        if x.shape != out.shape or {x.dtype, out.dtype} != {self.dtype}:
            raise KernelError(f"relu_squared: needs two {self.dtype} tensors of one shape")
        if row_gate is not None:
            if row_gate.dtype != self.dtype or row_gate.dim() != 2 or row_gate.shape != (x.shape[0], 1):
                raise KernelError("relu_squared: the row gate is [rows, 1] of the compute dtype")
            ld_g = row_gate.stride(0)
        h = lib("moe")
        _check(h.kvad_relu_squared(self.code, _ptr(x), ld_x, _ptr(out), ld_o, _ptr(row_gate), ld_g, x.shape[0], x.shape[1], _stream()), h)

    # -- mixing over time channel by channel ---------------------------------------------------
    def residual_conv(self, x, taps, out, state, state_off: int, row_seq, row_pos, seq_starts, seq_slots, *, shift: bool = False) -> None:
        """out = x + (causal convolution over time per channel of x) with `taps` [channels, n]: the last tap meets the row
        itself, inputs before the step's rows come from the sequence's kept inputs (`state[slot, state_off:]` as
        [n - 1, channels], 32-bit), zeros before position 0.  `shift`: every sequence brings ONE row and the kept inputs
        are moved on by it in the same launch (otherwise `conv_keep` does that afterwards)."""
        _need_cuda(x, taps, out, state, row_seq, row_pos, seq_starts, seq_slots)
        ld_x, ld_o = _rows_view(x, "residual_conv input"), _rows_view(out, "residual_conv output")
        C, n_taps = taps.shape
        if ({x.dtype, taps.dtype, out.dtype} != {self.dtype} or not taps.is_contiguous() or x.shape != out.shape or x.shape[1] != C
                or state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] < state_off + (n_taps - 1) * C):
            raise KernelError(f"residual_conv: needs {self.dtype} rows and taps [channels, n] and a float32 state with room for the kept inputs")
        h = lib("channel_recurrence")
        _check(h.kvad_residual_conv(self.code, _ptr(x), ld_x, _ptr(taps), _ptr(out), ld_o, _ptr(state), state.stride(0), int(state_off),
                                    _ptr(row_seq), _ptr(row_pos), _ptr(seq_starts), _ptr(seq_slots), x.shape[0], C, n_taps, int(bool(shift)),
                                    _stream()), h)

    def conv_keep(self, x, n_taps: int, state, state_off: int, seq_starts, seq_slots, n_seqs: int) -> None:
        """Keeps every sequence's last `n_taps` - 1 rows of x (older ones from what was kept) for the next step."""
        _need_cuda(x, state, seq_starts, seq_slots)
        ld_x, C = _rows_view(x, "conv_keep input"), x.shape[1]
        if x.dtype != self.dtype or state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] < state_off + (n_taps - 1) * C:
            raise KernelError("conv_keep: rows of the compute dtype and a float32 state with room for the kept inputs")
        h = lib("channel_recurrence")
        _check(h.kvad_conv_keep(self.code, _ptr(x), ld_x, _ptr(state), state.stride(0), int(state_off), _ptr(seq_starts), _ptr(seq_slots),
                                int(n_seqs), C, int(n_taps), _stream()), h)

    @staticmethod
    def min_gru_chunks(max_new: int) -> int:
        """Into how many chunks, walked side by side, the minGRU cuts a sequence's rows of a step: by the longest run of
        new rows only (one row: one chunk; from 16 rows a chunk on, up to 32 chunks)."""
        return max(1, min(32, max_new // 16))

    def min_gru(self, zug, width: int, out, state, seq_starts, seq_slots, n_seqs: int, max_new: int, *, state_off: int = 0) -> None:
        """Per sequence and channel over the step's rows in order: S = (1 - z) S + z c with z = sigmoid(a), c = u + 1/2 where
        u >= 0 and sigmoid(u) where u < 0; out = S * silu(g).  `zug` float32 [rows, 3 width] = a | u | g; `state` float32
        [slots, >= state_off + width] is carried on."""
        _need_cuda(zug, out, state, seq_starts, seq_slots)
        ld, ld_o = _rows_view(zug, "min_gru projections"), _rows_view(out, "min_gru output")
        if (zug.dtype != torch.float32 or zug.shape[1] < 3 * width or out.dtype != self.dtype or out.shape != (zug.shape[0], width)
                or state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] < state_off + width):
            raise KernelError(f"min_gru: float32 projections [rows, 3 width], {self.dtype} output [rows, width], float32 state")
        h = lib("channel_recurrence")
        _check(h.kvad_min_gru(self.code, _ptr(zug), ld, 0, int(width), 2 * int(width), _ptr(out), ld_o, _ptr(state), state.stride(0),
                              int(state_off), _ptr(seq_starts), _ptr(seq_slots), int(n_seqs), int(width), self.min_gru_chunks(max_new),
                              _stream()), h)

    # -- sampling ------------------------------------------------------------------
    ARGMAX_CHUNK = 2048

    def argmax(self, logits, out, scratch=None) -> None:
        """out[r] = first index of the largest logit of row r.  With `scratch` (int64, rows x
        ceil(vocab / 2048) words) the rows are reduced by many blocks each, in two stages."""
        _need_cuda(logits, out, scratch)
        ld = _rows_view(logits, "argmax logits")
        n, vocab = logits.shape
        if logits.dtype != torch.float32 or out.dtype != torch.int32 or out.numel() < n:
            raise KernelError("argmax: logits must be float32 and the output int32, one per row")
        if scratch is not None and (scratch.dtype != torch.int64 or scratch.numel() < n * -(-vocab // self.ARGMAX_CHUNK)):
            raise KernelError("argmax: scratch must be int64 with rows x ceil(vocab / 2048) words")
        h = lib("sampling")
        _check(h.kvad_argmax(_ptr(logits), ld, n, vocab, _ptr(out), _ptr(scratch), _stream()), h)
        if scratch is not None:
            global _launches
            _launches += 1

    def sample(self, logits, temperature, top_k, top_p, uniform, out) -> None:
        """out[r] = token for row r: greedy where temperature[r] <= 0, else top-k, softmax at
        temperature, top-p, and the draw uniform[r] in [0, 1)."""
        _need_cuda(logits, temperature, top_k, top_p, uniform, out)
        ld = _rows_view(logits, "sample logits")
        n = logits.shape[0]
        ok = (logits.dtype == torch.float32 and temperature.dtype == torch.float32 and top_p.dtype == torch.float32
              and top_k.dtype == torch.int32 and uniform.dtype == torch.float32 and out.dtype == torch.int32
              and min(temperature.numel(), top_k.numel(), top_p.numel(), uniform.numel(), out.numel()) >= n)
        if not ok:
            raise KernelError("sample: needs float32 logits/temperature/top_p/uniform and int32 top_k/out, one per row")
        h = lib("sampling")
        _check(h.kvad_sample(_ptr(logits), ld, n, logits.shape[1], _ptr(temperature), _ptr(top_k), _ptr(top_p),
                             _ptr(uniform), _ptr(out), _stream()), h)


def sample_force_general(on: bool) -> None:
    """Tests: True sends every sampling row through the selections over the whole vocabulary, also
    where a small top-k has a shorter way."""
    switches_changed()
    h = lib("sampling")
    h.kvad_sample_force_general.argtypes = [c_int]
    h.kvad_sample_force_general.restype = None
    h.kvad_sample_force_general(int(bool(on)))


def prefill_force_legacy(on: bool) -> None:
    """Tests: True keeps the prompt attention of head sizes 64 and 128 on the mma.sync kernel, not the tcgen05 one."""
    switches_changed()
    h = lib("attention_prefill")
    h.kvad_attention_prefill_force_legacy.argtypes = [c_int]
    h.kvad_attention_prefill_force_legacy.restype = None
    h.kvad_attention_prefill_force_legacy(int(bool(on)))


def prefill_split_above(pages: int) -> None:
    """Tests and measurements: the tensor-core prompt attention gives a tile of 128 rows to both slots of a CTA,
    half of its pages each, when it sees more than `pages` pages (0: the kernel's own choice, 8)."""
    h = lib("attention_prefill")
    h.kvad_attention_prefill_split_above.argtypes = [c_int]
    h.kvad_attention_prefill_split_above.restype = None
    h.kvad_attention_prefill_split_above(int(pages))
    switches_changed()


def prefill_wait_timeouts() -> int:
    """How many bounded waits of the tcgen05 prompt attention have run out (0 in a healthy run)."""
    h = lib("attention_prefill")
    h.kvad_attention_prefill_status.argtypes = []
    h.kvad_attention_prefill_status.restype = c_int
    n = h.kvad_attention_prefill_status()
    if n < 0:
        raise KernelError(h.kvad_last_error().decode("utf-8", "replace"))
    return n


def decode_force_plain(on) -> None:
    """Tests: 1 / True keeps the decode attention of every head size on the kernel that loads through
    registers; 2 keeps the TMA-fed kernel but merges splits through global memory, not a cluster; 0: default."""
    switches_changed()
    h = lib("attention_decode")
    h.kvad_attention_decode_force_plain.argtypes = [c_int]
    h.kvad_attention_decode_force_plain.restype = None
    h.kvad_attention_decode_force_plain(int(on))


def decode_wait_timeouts() -> int:
    """How many bounded waits of the TMA-fed decode attention have run out (0 in a healthy run)."""
    h = lib("attention_decode")
    h.kvad_attention_decode_status.argtypes = []
    h.kvad_attention_decode_status.restype = c_int
    n = h.kvad_attention_decode_status()
    if n < 0:
        raise KernelError(h.kvad_last_error().decode("utf-8", "replace"))
    return n


def tcgen05_load_form(mode: int) -> None:
    """Tests: 0 lets the swapped linear kernel choose between one TMA load per K block and grouped
    three-dimensional loads; 1 forces the former, 2 the latter (where K is a multiple of 64)."""
    switches_changed()
    h = lib("linear_tcgen05")
    h.kvad_linear_tcgen05_no_3d.argtypes = [c_int]
    h.kvad_linear_tcgen05_no_3d.restype = None
    h.kvad_linear_tcgen05_no_3d(int(mode))


def tcgen05_cluster_k(on: bool) -> None:
    """Tests: False keeps K whole under the storing epilogues of the swapped form (no reduction inside a cluster)."""
    switches_changed()
    h = build.load("linear_tcgen05")
    h.kvad_linear_tcgen05_no_cluster_k.argtypes = [c_int]
    h.kvad_linear_tcgen05_no_cluster_k.restype = None
    h.kvad_linear_tcgen05_no_cluster_k(int(not on))


def tcgen05_plain_stores(on: bool) -> None:
    """Tests: the wide linear kernel writes its output with plain stores instead of TMA stores / reduce-adds."""
    switches_changed()
    h = lib("linear_tcgen05")
    h.kvad_linear_tcgen05_no_tma_out.argtypes = [c_int]
    h.kvad_linear_tcgen05_no_tma_out.restype = None
    h.kvad_linear_tcgen05_no_tma_out(int(bool(on)))


def tcgen05_test_hooks(wait_limit: int = 0, skip_first_load: bool = False) -> None:
    """Tests of the bounded waits of the tensor-core linear kernel: `wait_limit` polls before a wait gives up
    (0: the library's own limit); `skip_first_load`: the next launch of the swapped form (17..64 rows) leaves
    out its first load, so its wait for it runs out and the launch returns with the status counter raised."""
    h = lib("linear_tcgen05")
    h.kvad_linear_tcgen05_test_hooks.argtypes = [ctypes.c_uint, c_int]
    h.kvad_linear_tcgen05_test_hooks.restype = c_int
    if h.kvad_linear_tcgen05_test_hooks(int(wait_limit), int(bool(skip_first_load))) != 0:
        raise KernelError(h.kvad_last_error().decode("utf-8", "replace"))


def tcgen05_wait_timeouts() -> int:
    """How many bounded waits of the tensor-core linear kernel have run out (0 in a healthy run)."""
    h = lib("linear_tcgen05")
    n = h.kvad_linear_tcgen05_status()
    if n < 0:
        raise KernelError(h.kvad_last_error().decode("utf-8", "replace"))
    return n


def tcgen05_takes(a, weight, out, lda: int, ldo: int) -> bool:
    """Shapes the tensor-core linear kernel accepts: TMA wants 16-byte aligned
    bases and row strides (bfloat16: multiples of 8 elements)."""
    k = a.shape[1]
    return (k % 8 == 0 and lda % 8 == 0 and a.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and out.data_ptr() % 16 == 0)
