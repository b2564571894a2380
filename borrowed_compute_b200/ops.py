"""Python faces of the CUDA launchers: argument checks, then one call into the kernel library.

Every function launches on torch's current CUDA stream and allocates nothing unless it
says so.  There is no CPU path and no library stand-in: a tensor that is not on a CUDA
device, or a kernel library that cannot be loaded, raises.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from .csrc import build as _build

PAGE = 64  # tokens per cache page; checked against the library at load

EPI_STORE, EPI_STORE_F32, EPI_ADD_F32, EPI_SWIGLU, EPI_RELU2 = 0, 1, 2, 3, 4

_c_int, _c_float, _c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


class KernelError(RuntimeError):
    pass


_checked_page = False


def lib() -> ctypes.CDLL:
    global _checked_page
    handle = _build.load()
    if not _checked_page:
        handle.bc_page_size.restype = _c_int
        if handle.bc_page_size() != PAGE:
            raise KernelError(f"the kernel library pages {handle.bc_page_size()} tokens, the package {PAGE}")
        _checked_page = True
        if os.environ.get("BC_B200_PDL", "1") == "0":
            handle.bc_set_pdl(_c_int(0))
        if os.environ.get("BC_B200_TC_STAGES"):        # measurement knob: cap the GEMM's TMA ring depth
            handle.bc_gemm_tc_set_stage_cap(_c_int(int(os.environ["BC_B200_TC_STAGES"])))
    return handle


def set_pdl(on: bool) -> None:
    """Whether kernels ask for programmatic dependent launch (overlap of a kernel's set-up
    and weight prefetch with the preceding kernel's tail).  On by default."""
    lib().bc_set_pdl(_c_int(1 if on else 0))


def set_gemm_tc_cluster(on: bool) -> None:
    """Whether two to eight splits of a product with few tokens add up inside a thread-block
    cluster (the default) or through scratch memory like all other splits; both give the same
    bits.  For measurements and tests."""
    lib().bc_gemm_tc_set_cluster(_c_int(1 if on else 0))


def set_gemm_tc_pair(on: bool) -> None:
    """Whether products over more than 128 tokens run on pairs of SMs that share a tile
    (cta_group::2, the default) or every block on its own.  For measurements and tests."""
    lib().bc_gemm_tc_set_pair(_c_int(1 if on else 0))


def set_gemm_tc_pair_tokens(n: int) -> None:
    """Tokens a tile of the paired product takes: 0 lets the launcher choose (256 unless a
    narrower tile saves a whole round of tiles), 64, 128, 192 or 256 force it."""
    lib().bc_gemm_tc_set_pair_tokens(_c_int(int(n)))


def _stream() -> _c_void_p:
    return _c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> _c_void_p:
    return _c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def _sink_values(sink: Optional[torch.Tensor], heads: int, who: str) -> None:
    """A softmax's learned sinks: float32, one number a head (or None)."""
    if sink is not None:
        _need(sink, "sink", torch.float32)
        if sink.numel() != heads:
            raise KernelError(f"{who}: {sink.numel()} sink values for {heads} heads")


def _suffix(dtype: torch.dtype) -> str:
    if dtype == torch.float32:
        return "f32"
    if dtype == torch.bfloat16:
        return "bf16"
    raise KernelError(f"no kernels for {dtype}: float32 and bfloat16 only")


# ------------------------------------------------------------------ the bounds-checked mode
# With BC_B200_BOUNDS_CHECK=1 (or ``bounds_check = True``) every launcher that takes indices
# (tokens, slots, positions, page tables, gathered rows) first brings them to the host and
# holds each against the extent of what it indexes; a bad one raises KernelError naming the
# tensor, the index and the extent, and nothing is launched.  The kernels themselves guard
# tokens, slots and pages on every build; this mode also catches what they would only skip
# (a position past the table, a gathered row past the rows) and what they trust (a slot past
# the table's rows).  It synchronises on every launch, so it is for finding a fault, not for
# serving; an engine built in this mode steps without captured graphs.  It stands in for a
# memory checker run under the kernels, which cannot be had everywhere.
bounds_check = os.environ.get("BC_B200_BOUNDS_CHECK", "0") == "1"


def _bounds(what: str, values: Optional[torch.Tensor], extent: int, count: Optional[int] = None, lowest: int = 0) -> None:
    """Every one of the first ``count`` values lies in [lowest, extent)."""
    if not bounds_check or values is None or torch.cuda.is_current_stream_capturing():
        return
    v = values.reshape(-1)[: values.numel() if count is None else count]
    if v.numel() == 0:
        return
    bad = ((v < lowest) | (v >= extent)).nonzero()
    if bad.numel():
        i = int(bad[0])
        raise KernelError(f"bounds check: {what}[{i}] = {int(v[i])} is outside [{lowest}, {extent})")


def _bounds_paged(who: str, rows: int, row_pos: torch.Tensor, row_slot: torch.Tensor, page_table: torch.Tensor, n_pages: int) -> None:
    """Slots name rows of the page table (or are -1: padding), positions fit the table's
    width, and every page the table names exists."""
    if not bounds_check or torch.cuda.is_current_stream_capturing():
        return
    _bounds(f"{who}: row_slot", row_slot, page_table.shape[0], rows, lowest=-1)
    live = row_slot.reshape(-1)[:rows] >= 0
    _bounds(f"{who}: row_pos", row_pos.reshape(-1)[:rows][live], page_table.shape[1] * PAGE)
    _bounds(f"{who}: page_table", page_table, n_pages, lowest=-1)


launches = 0   # kernels launched through this module since import (a captured graph replays them uncounted)
_KERNELS_PER_CALL = {"bc_argmax": 2, "bc_moe_plan": 3, "bc_moe_route_f32": 2, "bc_moe_route_bf16": 2}   # launchers that start more than one kernel


# Timing of single launches, for engine.profile.StepProfile: while `timeline` is a list every
# call records CUDA events around itself and appends (class, launcher, start, end).  The
# class is `label` if a part set one for the product it is about to run, else the launcher's.
timeline: Optional[list] = None
label = ""
_CLASS_OF = {
    "bc_embed": "embedding", "bc_rmsnorm": "norm", "bc_swiglu": "activation", "bc_rope_append": "rotary + append",
    "bc_attention_rows": "attention", "bc_attention_decode": "attention", "bc_attention_prefill": "attention",
    "bc_short_conv": "short convolution", "bc_norm_pair": "norm", "bc_delta": "delta rule", "bc_polynorm": "activation", "bc_qkv_prepare": "rotary + append",
    "bc_linear_scan": "recurrence", "bc_ssd_prepare": "recurrence set-up", "bc_gla_decay": "recurrence set-up", "bc_gated_norm": "gated norm",
    "bc_moe_product": "expert product", "bc_gemm_tc_grouped": "expert product", "bc_moe_route": "routing", "bc_moe_plan": "expert sort",
    "bc_moe_gather": "expert gather", "bc_moe_combine": "expert sum", "bc_softcap": "softcap", "bc_reentry": "re-entry",
    "bc_argmax": "sampling", "bc_sample": "sampling", "bc_gemm": "product", "bc_random": "random weights",
    "bc_latent_prepare": "latent norm + append", "bc_latent_query": "latent query", "bc_latent_rows": "attention", "bc_latent_decode": "attention", "bc_latent_heads": "latent query",
    "bc_latent_gather": "latent keys and values", "bc_latent_spread": "latent keys and values", "bc_latent_gate": "latent values",
    "bc_latent_values": "latent values", "bc_norm_add": "norm", "bc_relu2": "activation", "bc_glu_clipped": "activation",
    "bc_talk_prepare": "talk prepare", "bc_talk_rows": "talking attention", "bc_talk_tiles": "talking attention", "bc_scale": "softcap", "bc_add_bias": "bias", "bc_gated_add": "gated sum", "bc_moe_table_route": "routing",
}


def _class_of(name: str) -> str:
    if label:
        return label
    for prefix, cls in _CLASS_OF.items():
        if name.startswith(prefix):
            return cls
    return name


def _call(fn, *args) -> None:
    global launches
    launches += _KERNELS_PER_CALL.get(fn.__name__, 1)
    if timeline is not None:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        status = fn(*args)
        end.record()
        timeline.append((_class_of(fn.__name__), fn.__name__, start, end))
    else:
        status = fn(*args)
    if status != 0:
        msg = lib().bc_last_error()
        raise KernelError(f"{fn.__name__} failed ({status}): {msg.decode() if msg else ''}")


def _fn(name: str):
    f = getattr(lib(), name)
    f.restype = _c_int
    return f


# ---------------------------------------------------------------------------------- row-wise

def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[r, :] = table[tokens[r], :] * scale, widened to float32."""
    _need(table, "table")
    _need(tokens, "tokens", torch.int32)
    _need(out, "out", torch.float32)
    rows, (V, E) = tokens.numel(), table.shape
    if out.shape != (rows, E):
        raise KernelError(f"embed: out is {tuple(out.shape)}, wanted {(rows, E)}")
    _bounds("embed: tokens", tokens, V)
    _call(_fn("bc_embed_" + _suffix(table.dtype)), _ptr(table), _ptr(tokens), _ptr(out), _c_int(rows), _c_int(E), _c_int(V), _c_float(scale), _stream())


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float, gather: Optional[torch.Tensor] = None) -> None:
    """out[i] = x[gather[i] or i] * rsqrt(mean(x^2) + eps) * weight; x and weight float32."""
    _need(x, "x", torch.float32)
    _need(weight, "weight", torch.float32)
    _need(out, "out")
    E = x.shape[-1]
    rows = out.shape[0]
    if weight.numel() != E or out.shape[-1] != E:
        raise KernelError(f"rmsnorm: widths differ: x {E}, weight {weight.numel()}, out {out.shape[-1]}")
    if gather is not None:
        _need(gather, "gather", torch.int32)
        if gather.numel() != rows:
            raise KernelError("rmsnorm: gather and out differ in rows")
        _bounds("rmsnorm: gather", gather, x.shape[0])
    elif x.shape[0] != rows:
        raise KernelError("rmsnorm: x and out differ in rows")
    _call(_fn("bc_rmsnorm_" + _suffix(out.dtype)), _ptr(x), _ptr(weight), _ptr(out), _ptr(gather), _c_int(rows), _c_int(E),
          _c_float(eps), _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[r, j] = silu(gate_up[r, j]) * gate_up[r, F + j]."""
    _need(gate_up, "gate_up")
    _need(out, "out", gate_up.dtype)
    rows, F = out.shape
    if gate_up.shape != (rows, 2 * F):
        raise KernelError(f"swiglu: gate_up is {tuple(gate_up.shape)}, wanted {(rows, 2 * F)}")
    _call(_fn("bc_swiglu_" + _suffix(out.dtype)), _ptr(gate_up), _ptr(out), _c_int(rows), _c_int(F), _stream())


def rope_append(qkv: torch.Tensor, cos_sin: Optional[torch.Tensor], row_pos: torch.Tensor, row_slot: torch.Tensor,
                page_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                pairing: int, write_cache: bool = True) -> None:
    """Rotates q and k of the fused projection in place by each row's position and writes
    rotated k and v into the row's cache page.  k_cache, v_cache: [pages, kv_heads, PAGE, head_dim]."""
    _need(qkv, "qkv")
    _need(row_pos, "row_pos", torch.int32)
    _need(row_slot, "row_slot", torch.int32)
    _need(page_table, "page_table", torch.int32)
    _need(k_cache, "k_cache", qkv.dtype)
    _need(v_cache, "v_cache", qkv.dtype)
    rows = qkv.shape[0]
    if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
        raise KernelError(f"rope_append: qkv width {qkv.shape[1]} is not (heads + 2 kv_heads) * head_dim")
    if row_pos.numel() < rows or row_slot.numel() < rows:
        raise KernelError("rope_append: fewer positions or slots than rows")
    n_pages = k_cache.shape[0]
    if tuple(k_cache.shape[1:]) != (kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"rope_append: cache is {tuple(k_cache.shape)}, wanted [pages, {kv_heads}, {PAGE}, {head_dim}]")
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32)
        if tuple(cos_sin.shape[1:]) != (head_dim // 2, 2):
            raise KernelError(f"rope_append: cos_sin is {tuple(cos_sin.shape)}, wanted [positions, {head_dim // 2}, 2]")
    _bounds_paged("rope_append", rows, row_pos, row_slot, page_table, n_pages)
    if cos_sin is not None and bounds_check and not torch.cuda.is_current_stream_capturing():
        _bounds("rope_append: row_pos (against the rotary table)", row_pos.reshape(-1)[:rows][row_slot.reshape(-1)[:rows] >= 0], cos_sin.shape[0])
    _call(_fn("bc_rope_append_" + _suffix(qkv.dtype)), _ptr(qkv), _ptr(cos_sin), _ptr(row_pos), _ptr(row_slot), _ptr(page_table),
          _ptr(k_cache), _ptr(v_cache), _c_int(rows), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(pairing),
          _c_int(page_table.shape[1]), _c_int(n_pages), _c_int(1 if write_cache else 0), _stream())


def random_normal(out: torch.Tensor, key: int, std: float) -> None:
    """out[i] = std * z(key, i) over out's elements in memory order: z a standard normal
    deviate that depends on the 64-bit key and the index alone (weights/random_init.py has
    the host's mirror, which gives the same bits)."""
    _need(out, "out")
    _call(_fn("bc_random_normal_" + _suffix(out.dtype)), _ptr(out), ctypes.c_longlong(out.numel()), ctypes.c_ulonglong(key & ((1 << 64) - 1)),
          _c_float(std), _stream())


# ---------------------------------------------------------------------------------- products

def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int) -> None:
    """out = x @ w.T on the CUDA cores with float accumulation in ascending k.
    EPI_STORE: out in x's type; EPI_STORE_F32: float32; EPI_ADD_F32: out += (float32);
    EPI_SWIGLU: w stacks gate rows on up rows, out[:, j] = silu(g_j) * u_j in x's type;
    EPI_RELU2: out = max(sum, 0)^2 in x's type, squared in float and rounded once."""
    _need(x, "x")
    _need(w, "w", x.dtype)
    M, K = x.shape
    n_w = w.shape[0]
    N = n_w // 2 if epilogue == EPI_SWIGLU else n_w
    if w.shape[1] != K or (epilogue == EPI_SWIGLU and n_w % 2):
        raise KernelError(f"gemm: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    _need(out, "out", torch.float32 if epilogue in (EPI_STORE_F32, EPI_ADD_F32) else x.dtype)
    if tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: out is {tuple(out.shape)}, wanted {(M, N)}")
    _call(_fn("bc_gemm_simt_" + _suffix(x.dtype)), _ptr(x), _ptr(w), _ptr(out), _c_int(M), _c_int(N), _c_int(K), _c_int(epilogue), _stream())


def sm_count() -> int:
    """Streaming multiprocessors of the current device, as the kernel library sees them."""
    return int(_fn("bc_sm_count")())


_tc_workspace = {}
_TC_FILL = float(os.environ.get("BC_B200_TC_FILL", "2"))      # measurement knobs: blocks an SM a split product aims at,
_SWIGLU_SPLIT = os.environ.get("BC_B200_SWIGLU_SPLIT", "1") == "1"
_TC_MIN_K = int(os.environ.get("BC_B200_TC_MIN_K", "4"))       # and the fewest k-steps of 64 a split keeps
TC_SCRATCH_FLOATS = 148 * 256 * 256   # split-K partial tiles: a capacity of 37 MiB (148 tiles of 256 x 256 floats), whatever the device


def _tc_scratch(device: torch.device):
    """Split-K scratch of the tensor-core product, one a device, allocated at first use:
    float partial tiles (any contents) and int counters (zero between launches)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _tc_workspace:
        _tc_workspace[key] = (torch.empty(TC_SCRATCH_FLOATS, dtype=torch.float32, device=device),
                              torch.zeros(4096, dtype=torch.int32, device=device))
    return _tc_workspace[key]


def gemm_tc_accepts(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core product takes these operands (K a multiple of 8, bf16)."""
    return x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def _tc_tiling(T: int, N: int, epilogue: int):
    """(token tile, output rows a block, blocks) the tensor-core product uses; mirrors the launcher."""
    bn = int(_fn("bc_gemm_tc_token_tile")(_c_int(T), _c_int(epilogue)))
    rows = int(_fn("bc_gemm_tc_rows_per_block")(_c_int(T), _c_int(N), _c_int(epilogue)))
    return bn, rows, -(-N // rows) * -(-T // bn)


def gemm_tc_splits(T: int, N: int, K: int, epilogue: int) -> int:
    """How many ways to split K so that a product with few weight tiles still fills the
    device's SMs: as many as fit, each at least 4 k-steps of 64 (8 measured 3 % slower on the
    3B shape, whose products of K = 3,072 then stopped at 4 splits, and 0.6 % on the 8B shape)."""
    bn, rows, tiles = _tc_tiling(T, N, epilogue)
    if tiles == 0:
        return 1
    sms = sm_count()
    accs = 2 if epilogue == EPI_SWIGLU else 1              # SwiGLU keeps gate and up sums apart until the last split
    fits = TC_SCRATCH_FLOATS // (tiles * accs * rows * bn)   # splits whose partial tiles fit the scratch
    if epilogue == EPI_SWIGLU:
        # The kernel can split SwiGLU (the gate is applied to the full sums), but measured on the
        # 8B shapes two half-depth blocks an SM stream slower than one full-depth block: unsplit,
        # unless the tiles are so few that they leave half of the SMs or more without a block
        # (a feed-forward width of 8,192 is 64 tiles): then one block an SM.
        if bn <= 64 and tiles * 2 <= sms and _SWIGLU_SPLIT:
            s = max(1, min(sms // tiles, -(-K // 64) // _TC_MIN_K, 8, fits))   # two blocks an SM measured slower here too
            return 1 << (s.bit_length() - 1)
        return 1
    if bn <= 64:
        # Few tokens: the product streams weights, two blocks fit an SM, and measured rates keep
        # rising up to about two blocks an SM as long as a split still has a few k-steps of 64.
        s = max(1, min(int(_TC_FILL * sms) // tiles, -(-K // 64) // _TC_MIN_K, 16, fits))
        # Up to eight splits add up inside a thread-block cluster, which saves the trip through
        # scratch memory; clusters of 2, 4 or 8 place well on the SMs, other sizes measured
        # up to 5 us slower.  So a count up to 12 is rounded down to a power of two.
        if s <= 12:
            s = 1 << (min(s, 8).bit_length() - 1)
        return s
    return max(1, min(sms // tiles, -(-K // 64) // 8, 16, fits))


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int, splits: Optional[int] = None,
            glu: Optional[Tuple[float, float]] = None) -> None:
    """out = x @ w.T for bf16 operands on the tcgen05 tensor cores (float accumulation in
    TMEM), with the epilogues of gemm_simt.  ``splits`` > 1 cuts K across blocks that add
    their partial sums in a fixed order.  ``glu`` = (limit, alpha) turns EPI_SWIGLU's gate into the bounded one:
    out = g' sigmoid(alpha g') (u' + 1) with g' = min(g, limit), u' = clamp(u, -limit, limit)."""
    _need(x, "x", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    M, K = x.shape
    n_w = w.shape[0]
    N = n_w // 2 if epilogue == EPI_SWIGLU else n_w
    if w.shape[1] != K or (epilogue == EPI_SWIGLU and n_w % 2):
        raise KernelError(f"gemm: x is {tuple(x.shape)}, w is {tuple(w.shape)}")
    _need(out, "out", torch.float32 if epilogue in (EPI_STORE_F32, EPI_ADD_F32) else torch.bfloat16)
    if tuple(out.shape) != (M, N):
        raise KernelError(f"gemm: out is {tuple(out.shape)}, wanted {(M, N)}")
    if M == 0:
        return
    if splits is None:
        splits = gemm_tc_splits(M, N, K, epilogue)
    partial = counters = None
    if splits > 1:
        partial, counters = _tc_scratch(x.device)
        bn, rows, tiles = _tc_tiling(M, N, epilogue)
        accs = 2 if epilogue == EPI_SWIGLU else 1
        if tiles * splits * accs * rows * bn > partial.numel() or tiles * 4 > counters.numel():
            raise KernelError(f"gemm_tc: {tiles} tiles are too many for the split-K scratch; use splits=1")
    if glu is not None:
        # The gated product with bounds (limit, alpha): out = g' sigmoid(alpha g') (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit).
        if epilogue != EPI_SWIGLU:
            raise KernelError("gemm_tc: bounds come with the gated product (EPI_SWIGLU)")
        _call(_fn("bc_gemm_tc_glu_bf16"), _ptr(x), _ptr(w), _ptr(out), _c_int(M), _c_int(N), _c_int(K), _c_int(splits), _ptr(partial), _ptr(counters),
              _c_float(glu[0]), _c_float(glu[1]), _stream())
        return
    _call(_fn("bc_gemm_tc_bf16"), _ptr(x), _ptr(w), _ptr(out), _c_int(M), _c_int(N), _c_int(K), _c_int(epilogue), _c_int(splits),
          _ptr(partial), _ptr(counters), _stream())


def gemm_tc_status(reset: bool = True) -> int:
    """Waits for the device and returns the tensor-core kernels' status word: 0, or
    (code << 16 | block) of the first bounded wait that gave up."""
    return int(_fn("bc_gemm_tc_status")(_c_int(1 if reset else 0)))


def set_wait_cycles(cycles: int = 0) -> None:
    """The most clocks a bounded wait inside the tensor-core kernels may take before it gives
    up and records its status (0: back to the default, about a second)."""
    for unit in ("gemm_tc", "attention_prefill_tc", "attention_decode"):
        st = _fn(f"bc_{unit}_set_wait_cycles")(ctypes.c_longlong(int(cycles)))
        if st != 0:
            raise KernelError(f"setting the wait limit of {unit} failed ({st})")


def gemm_tc_test_starve_next_launch() -> None:
    """Test hook: the next product of at most 128 tokens waits for bytes that never come, so
    that one of its bounded waits runs out (see csrc/gemm_tc.cu).  Its output stays unwritten."""
    lib().bc_gemm_tc_test_starve_next_launch()


# ------------------------------------------------------------ errors that reach the caller

_STATUS_UNITS = ("the tensor-core product (gemm_tc)", "the tcgen05 prompt attention (attention_prefill_tc)", "the decode attention (attention_decode)")
_WAITS = {
    0: {1: "the loader's wait for a free stage", 2: "the wait for a stage's operands", 3: "the epilogue's wait for the accumulator",
        4: "the wait for the epilogue to hand the accumulator back"},
    1: {1: "the loader's wait for a free stage", 2: "the wait for the queries", 3: "the wait for the first pages", 4: "the wait for P",
        5: "the wait for a page", 6: "the softmax's wait for scores", 7: "the wait for a product that frees P", 8: "the wait for the last product",
        9: "the wait before a rescale"},
    2: {1: "the wait for a page of keys and values"},
}
_bound_devices = set()


def bind_status(device: Optional[torch.device] = None) -> None:
    """Gives the kernels of ``device`` their words of host-visible memory (once a device), so
    that check_status can look without waiting for the device."""
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    if index in _bound_devices:
        return
    with torch.cuda.device(index):
        _call(_fn("bc_status_bind"))
    _bound_devices.add(index)


def check_status(device: Optional[torch.device] = None) -> None:
    """Raises KernelError if a bounded wait of a kernel gave up since the last look.  Costs a
    read of host memory; meaningful after the caller has synchronised with the device (the
    word is written by the kernel that gave up, before it ends).  The word is cleared, so
    the next look reports only what happens after this one."""
    index = torch.cuda.current_device() if device is None or device.index is None else device.index
    if index not in _bound_devices:
        return
    peek = _fn("bc_status_peek")
    with torch.cuda.device(index):
        for unit, name in enumerate(_STATUS_UNITS):
            word = int(peek(_c_int(unit), _c_int(1)))
            if word != 0:
                code, block = word >> 16, word & 0xFFFF
                raise KernelError(f"{name}: {_WAITS[unit].get(code, 'a wait')} (code {code}) ran out in block {block}; "
                                  f"what that launch should have written is missing, so this step's results are not valid")


_self_checked = set()


def self_check(device: torch.device) -> None:
    """Once a device and process: every epilogue of the tensor-core product, and the CUDA-core
    product, on a 37 x 512 weight with one row and with three, against float64 sums, as the
    reference checks its products before it trusts a GPU (crates/bc-infer/src/gpu/mod.rs:
    181-206, same sizes, same inputs rule, same 1e-3 (1 + |want|) bound; there a failure means
    the CPU serves, here there is no other path, so it raises)."""
    import numpy as np

    index = device.index if device.index is not None else torch.cuda.current_device()
    if index in _self_checked:
        return
    rows_w, cols = 37, 512
    rng = np.random.default_rng(7)
    w = rng.standard_normal((2 * rows_w, cols)).astype(np.float32) * 0.5
    wb = torch.from_numpy(w).to(device=device, dtype=torch.bfloat16)
    w64 = wb.float().cpu().numpy().astype(np.float64)

    def bad(got: torch.Tensor, want: np.ndarray, rel: float = 1e-3) -> bool:
        g = got.float().cpu().numpy().astype(np.float64)
        return (not np.isfinite(g).all()) or bool((np.abs(g - want) > rel * (1.0 + np.abs(want))).any())

    rounded = 2.0 ** -7    # an output that is itself rounded to bfloat16 carries half an ulp of 2^-8 besides
    for n in (1, 3):       # one row and a batch take different paths
        x = (((np.arange(n * cols) * 31 % 97).astype(np.float32) - 48.0) / 50.0).reshape(n, cols)
        xb = torch.from_numpy(x).to(device=device, dtype=torch.bfloat16)
        x64 = xb.float().cpu().numpy().astype(np.float64)
        full = x64 @ w64.T                                                    # [n, 74]: gate rows, then up rows
        gate, up = full[:, :rows_w], full[:, rows_w:]
        for name, product in (("tensor-core", gemm_tc), ("CUDA-core", gemm_simt)):
            stored = torch.empty((n, 2 * rows_w), dtype=torch.bfloat16, device=device)
            product(xb, wb, stored, EPI_STORE)
            scores = torch.empty((n, 2 * rows_w), dtype=torch.float32, device=device)
            product(xb, wb, scores, EPI_STORE_F32)
            added = torch.full((n, 2 * rows_w), 0.25, dtype=torch.float32, device=device)
            product(xb, wb, added, EPI_ADD_F32)
            gated = torch.empty((n, rows_w), dtype=torch.bfloat16, device=device)
            product(xb, wb, gated, EPI_SWIGLU)
            squared = torch.empty((n, 2 * rows_w), dtype=torch.bfloat16, device=device)
            product(xb, wb, squared, EPI_RELU2)
            checks = {"store": bad(stored, full, rounded), "store_f32": bad(scores, full), "add_f32": bad(added, full + 0.25),
                      "swiglu": bad(gated, gate / (1.0 + np.exp(-gate)) * up, rounded), "relu2": bad(squared, np.maximum(full, 0.0) ** 2, rounded)}
            wrong = [k for k, v in checks.items() if v]
            if wrong:
                raise KernelError(f"self-check: the {name} product with {n} row(s) is wrong for the epilogue(s) {wrong} on a "
                                  f"{rows_w} x {cols} weight; this device or this build of the kernels cannot be trusted")
    x = (((np.arange(3 * cols) * 31 % 97).astype(np.float32) - 48.0) / 50.0).reshape(3, cols)
    scores = torch.empty((3, 2 * rows_w), dtype=torch.float32, device=device)
    gemm_simt(torch.from_numpy(x).to(device), torch.from_numpy(w).to(device), scores, EPI_STORE_F32)
    if bad(scores, x.astype(np.float64) @ w.astype(np.float64).T):
        raise KernelError("self-check: the float32 CUDA-core product is wrong; this device or this build of the kernels cannot be trusted")
    torch.cuda.synchronize(device)
    check_status(device)
    _self_checked.add(index)


def set_attention_prefill_tc_tiles(n: int) -> None:
    """Query tiles (of 128 rows) a block of the tcgen05 prompt attention: 0 lets the launcher
    choose (two, unless no sequence brings more rows than one tile holds), 1 or 2 force it.
    For measurements and tests."""
    lib().bc_attention_prefill_tc_set_tiles(_c_int(int(n)))


def attention_prefill_tc_status(reset: bool = True) -> int:
    """The same word of the tcgen05 prompt attention kernel."""
    return int(_fn("bc_attention_prefill_tc_status")(_c_int(1 if reset else 0)))


# --------------------------------------------------------------------------------- attention

def attention_rows(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor,
                   row_pos: torch.Tensor, row_slot: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                   window: int = 0, scale: Optional[float] = None, value_dim: Optional[int] = None, chunk: int = 0, sink: bool = False,
                   out_scale: float = 1.0) -> None:
    """Causal attention of every row against its slot's cached positions, one warp a (row, head).
    ``sink`` adds one to the softmax's denominator (a position of score 0 without a value); ``out_scale`` multiplies the result.
    ``value_dim`` (default: ``head_dim``) is the width of a head's values, ``chunk`` > 0 lets a
    position see only those of its own chunk of that many positions, counted from position 0."""
    _need(q, "q")
    _need(k_cache, "k_cache", q.dtype)
    _need(v_cache, "v_cache", q.dtype)
    _need(page_table, "page_table", torch.int32)
    _need(row_pos, "row_pos", torch.int32)
    _need(row_slot, "row_slot", torch.int32)
    _need(out, "out", q.dtype)
    rows = out.shape[0]
    value_dim = head_dim if value_dim is None else int(value_dim)
    if out.shape[1] != heads * value_dim:
        raise KernelError(f"attention: out width {out.shape[1]} is not heads * value_dim")
    if tuple(k_cache.shape[1:]) != (kv_heads, PAGE, head_dim) or tuple(v_cache.shape) != (k_cache.shape[0], kv_heads, PAGE, value_dim):
        raise KernelError(f"attention: cache is {tuple(k_cache.shape)} and {tuple(v_cache.shape)}, wanted [pages, {kv_heads}, {PAGE}, "
                          f"{head_dim}] and [pages, {kv_heads}, {PAGE}, {value_dim}]")
    if scale is None:
        scale = 1.0 / float(head_dim) ** 0.5
    _bounds_paged("attention_rows", rows, row_pos, row_slot, page_table, k_cache.shape[0])
    _call(_fn("bc_attention_rows_sink_" + _suffix(q.dtype)), _ptr(q), _c_int(q_stride), _ptr(k_cache), _ptr(v_cache), _ptr(page_table),
          _ptr(row_pos), _ptr(row_slot), _ptr(out), _c_int(rows), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(value_dim),
          _c_int(page_table.shape[1]), _c_int(k_cache.shape[0]), _c_int(window), _c_int(chunk), _c_float(scale), _c_int(1 if sink else 0),
          _c_float(out_scale), _stream())


# ------------------------------------------------------- parts of other mixers and feed-forwards

def short_conv(h: torch.Tensor, weight_t: torch.Tensor, tail: torch.Tensor, seq_rows: torch.Tensor, seq_slot: torch.Tensor,
               out: torch.Tensor, seqs: int, max_new: int, write_tail: bool = True) -> None:
    """out = h + causal convolution of h over time on every channel; ``weight_t`` [taps, E] float32 (the kernel
    transposed: tap by tap), ``tail`` [slots, taps - 1, E] holds every slot's last inputs and is brought up to date."""
    _need(h, "h")
    _need(weight_t, "weight_t", torch.float32)
    _need(tail, "tail", h.dtype)
    _need(seq_rows, "seq_rows", torch.int32)
    _need(seq_slot, "seq_slot", torch.int32)
    _need(out, "out", h.dtype)
    taps, E = weight_t.shape
    if h.shape[-1] != E or out.shape != h.shape or tuple(tail.shape[1:]) != (taps - 1, E):
        raise KernelError(f"short_conv: h {tuple(h.shape)}, out {tuple(out.shape)}, tail {tuple(tail.shape)} do not fit weight {(taps, E)}")
    if h.data_ptr() == out.data_ptr():
        raise KernelError("short_conv: out must not be h (rows read their predecessors)")
    _bounds("short_conv: seq_slot", seq_slot, tail.shape[0], seqs, lowest=-1)
    _bounds("short_conv: seq_rows", seq_rows, h.shape[0] + 1, seqs + 1)
    _call(_fn("bc_short_conv_" + _suffix(h.dtype)), _ptr(h), _ptr(weight_t), _ptr(tail), _ptr(seq_rows), _ptr(seq_slot), _ptr(out),
          _c_int(seqs), _c_int(max_new), _c_int(E), _c_int(taps), _c_int(tail.shape[0]), _c_int(1 if write_tail else 0), _stream())


def norm_pair(x: torch.Tensor, w1: torch.Tensor, w2: Optional[torch.Tensor], out1: torch.Tensor, out2: Optional[torch.Tensor], eps: float,
              conv_weight: Optional[torch.Tensor] = None, tail: Optional[torch.Tensor] = None, row_slot: Optional[torch.Tensor] = None,
              write_tail: bool = True) -> None:
    """Two RMS norms of the same rows with one statistic: out1 = x / rms(x) * w1, out2 = x / rms(x) * w2 (the second
    may be left out).  With ``conv_weight`` [taps, E] (transposed, as for ``short_conv``) the first output also passes the short causal convolution of
    ``short_conv``, for steps in which every sequence brings one row (row r belongs to slot ``row_slot[r]``); the
    tail is brought up to date."""
    _need(x, "x", torch.float32)
    _need(w1, "w1", torch.float32)
    _need(out1, "out1")
    rows, E = x.shape
    if w1.numel() != E or tuple(out1.shape) != (rows, E):
        raise KernelError(f"norm_pair: x {tuple(x.shape)}, w1 {w1.numel()}, out1 {tuple(out1.shape)} do not fit")
    if (w2 is None) != (out2 is None):
        raise KernelError("norm_pair: the second norm needs its weight and its output")
    if w2 is not None:
        _need(w2, "w2", torch.float32)
        _need(out2, "out2", out1.dtype)
        if w2.numel() != E or out2.shape != out1.shape:
            raise KernelError("norm_pair: the second norm's sizes differ")
    taps, n_slots = 0, 0
    if conv_weight is not None:
        _need(conv_weight, "conv_weight", torch.float32)
        _need(tail, "tail", out1.dtype)
        _need(row_slot, "row_slot", torch.int32)
        taps, n_slots = conv_weight.shape[0], tail.shape[0]
        if conv_weight.shape[1] != E or tuple(tail.shape[1:]) != (taps - 1, E) or row_slot.numel() < rows:
            raise KernelError(f"norm_pair: conv weight {tuple(conv_weight.shape)}, tail {tuple(tail.shape)} do not fit {E} channels")
        _bounds("norm_pair: row_slot", row_slot, n_slots, rows, lowest=-1)
    _call(_fn("bc_norm_pair_" + _suffix(out1.dtype)), _ptr(x), _ptr(w1), _ptr(w2), _ptr(conv_weight), _ptr(tail), _ptr(row_slot), _ptr(out1),
          _ptr(out2), _c_int(rows), _c_int(E), _c_float(eps), _c_int(taps), _c_int(n_slots), _c_int(1 if write_tail else 0), _stream())


def delta_prepare(proj: torch.Tensor, w2t: torch.Tensor, w0: torch.Tensor, a_bias: torch.Tensor, decay: torch.Tensor, unit: torch.Tensor,
                  removal: torch.Tensor, dots: torch.Tensor, heads: int, head_dim: int, decay_scale: float, key_eps: float) -> None:
    """From the fused projection [rows, 5 H D + inner] (r, k, v, gate, a, decay's inner projection; float32): per key
    channel the decay exp(-decay_scale * sigmoid(w2 tanh(inner) + w0)), the key over its length, the removal
    rate sigmoid(a + a_bias) times that unit key, and per head the dot products r.(removal) and r.k.
    ``w2t`` is w2 transposed, [inner, H D]."""
    rows, stride = proj.shape
    HD = heads * head_dim
    inner = w2t.shape[0]
    for t, name in ((proj, "proj"), (w2t, "w2t"), (w0, "w0"), (a_bias, "a_bias"), (decay, "decay"), (unit, "unit"), (removal, "removal"), (dots, "dots")):
        _need(t, name, torch.float32)
    if w2t.shape[1] != HD or w0.numel() != HD or a_bias.numel() != HD or stride != 5 * HD + inner:
        raise KernelError(f"delta_prepare: proj {tuple(proj.shape)}, w2t {tuple(w2t.shape)} do not fit {heads} heads of {head_dim}")
    if any(tuple(t.shape) != (rows, HD) for t in (decay, unit, removal)) or tuple(dots.shape) != (rows, heads, 2):
        raise KernelError("delta_prepare: outputs must be [rows, H D] and dots [rows, H, 2]")
    _call(_fn("bc_delta_prepare"), _ptr(proj), _c_int(stride), _ptr(w2t), _ptr(w0), _ptr(a_bias), _ptr(decay), _ptr(unit), _ptr(removal),
          _ptr(dots), _c_int(rows), _c_int(heads), _c_int(head_dim), _c_int(inner), _c_float(decay_scale), _c_float(key_eps), _stream())


def delta_scan(proj: torch.Tensor, decay: torch.Tensor, unit: torch.Tensor, removal: torch.Tensor, dots: torch.Tensor, state: torch.Tensor,
               seq_rows: torch.Tensor, seq_slot: torch.Tensor, out: torch.Tensor, seqs: int, heads: int, head_dim: int,
               write_state: bool = True) -> None:
    """The recurrence S <- diag(decay) S - removal (unit^T S) + k v^T, o = S^T r over every sequence's rows in
    time order, from and into ``state`` [slots, H, D, D] float32; ``out`` [rows, H D] float32."""
    for t, name in ((proj, "proj"), (decay, "decay"), (unit, "unit"), (removal, "removal"), (dots, "dots"), (state, "state"), (out, "out")):
        _need(t, name, torch.float32)
    _need(seq_rows, "seq_rows", torch.int32)
    _need(seq_slot, "seq_slot", torch.int32)
    if tuple(state.shape[1:]) != (heads, head_dim, head_dim) or out.shape != decay.shape or proj.shape[1] < 3 * heads * head_dim:
        raise KernelError(f"delta_scan: state {tuple(state.shape)} or out {tuple(out.shape)} do not fit {heads} heads of {head_dim}")
    _bounds("delta_scan: seq_slot", seq_slot, state.shape[0], seqs, lowest=-1)
    _bounds("delta_scan: seq_rows", seq_rows, proj.shape[0] + 1, seqs + 1)
    _call(_fn("bc_delta_scan"), _ptr(proj), _c_int(proj.shape[1]), _ptr(decay), _ptr(unit), _ptr(removal), _ptr(dots), _ptr(state),
          _ptr(seq_rows), _ptr(seq_slot), _ptr(out), _c_int(seqs), _c_int(heads), _c_int(head_dim), _c_int(state.shape[0]),
          _c_int(1 if write_state else 0), _stream())


def delta_finish(o: torch.Tensor, proj: torch.Tensor, gate_offset: int, weight: torch.Tensor, out: torch.Tensor, heads: int, head_dim: int,
                 eps: float) -> None:
    """out = o / rms(o over each head) * weight * sigmoid(gate), the gate at columns gate_offset .. of ``proj``."""
    _need(o, "o", torch.float32)
    _need(proj, "proj", torch.float32)
    _need(weight, "weight", torch.float32)
    _need(out, "out")
    rows, HD = o.shape
    if HD != heads * head_dim or out.shape != o.shape or weight.numel() != HD or gate_offset + HD > proj.shape[1] or proj.shape[0] != rows:
        raise KernelError("delta_finish: shapes do not fit")
    gate = proj.reshape(-1)[gate_offset:]
    _call(_fn("bc_delta_finish_" + _suffix(out.dtype)), _ptr(o), _c_void_p(gate.data_ptr()), _c_int(proj.shape[1]), _ptr(weight), _ptr(out),
          _c_int(rows), _c_int(heads), _c_int(head_dim), _c_float(eps), _stream())


def delta_step_accepts(head_dim: int) -> bool:
    """Whether the one-launch step for single rows takes heads of this size (up to 128 channels)."""
    return 0 < head_dim <= 128


def delta_step(proj: torch.Tensor, w2t: torch.Tensor, w0: torch.Tensor, a_bias: torch.Tensor, norm_weight: torch.Tensor, state: torch.Tensor,
               row_slot: torch.Tensor, out: torch.Tensor, heads: int, head_dim: int, decay_scale: float, key_eps: float, norm_eps: float,
               write_state: bool = True) -> None:
    """``delta_prepare``, one step of ``delta_scan`` and ``delta_finish`` in one launch, for steps in which every
    sequence brings one row (row r lives in slot ``row_slot[r]``); the same bits as the three."""
    for t, name in ((proj, "proj"), (w2t, "w2t"), (w0, "w0"), (a_bias, "a_bias"), (norm_weight, "norm_weight"), (state, "state")):
        _need(t, name, torch.float32)
    _need(row_slot, "row_slot", torch.int32)
    _need(out, "out")
    rows, stride = proj.shape
    HD, inner = heads * head_dim, w2t.shape[0]
    if w2t.shape[1] != HD or w0.numel() != HD or a_bias.numel() != HD or norm_weight.numel() != HD or stride != 5 * HD + inner:
        raise KernelError(f"delta_step: proj {tuple(proj.shape)}, w2t {tuple(w2t.shape)} do not fit {heads} heads of {head_dim}")
    if tuple(state.shape[1:]) != (heads, head_dim, head_dim) or tuple(out.shape) != (rows, HD) or row_slot.numel() < rows:
        raise KernelError(f"delta_step: state {tuple(state.shape)} or out {tuple(out.shape)} do not fit")
    _bounds("delta_step: row_slot", row_slot, state.shape[0], rows, lowest=-1)
    _call(_fn("bc_delta_step_" + _suffix(out.dtype)), _ptr(proj), _c_int(stride), _ptr(w2t), _ptr(w0), _ptr(a_bias), _ptr(norm_weight),
          _ptr(state), _ptr(row_slot), _ptr(out), _c_int(rows), _c_int(heads), _c_int(head_dim), _c_int(inner), _c_float(decay_scale),
          _c_float(key_eps), _c_float(norm_eps), _c_int(state.shape[0]), _c_int(1 if write_state else 0), _stream())


def polynorm(z: torch.Tensor, coef: torch.Tensor, out: torch.Tensor, eps: float) -> None:
    """out = a N(z) + b N(z^2) + c N(z^3) + e with (a, b, c, e) = coef and N the division of a row by its root mean square."""
    _need(z, "z", torch.float32)
    _need(coef, "coef", torch.float32)
    _need(out, "out")
    if coef.numel() != 4 or out.shape != z.shape:
        raise KernelError(f"polynorm: coef has {coef.numel()} numbers (wanted 4) or out {tuple(out.shape)} is not z {tuple(z.shape)}")
    _call(_fn("bc_polynorm_" + _suffix(out.dtype)), _ptr(z), _ptr(coef), _ptr(out), _c_int(z.shape[0]), _c_int(z.shape[1]), _c_float(eps),
          _stream())


def qkv_prepare(qkv: torch.Tensor, bias: Optional[torch.Tensor], q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                cos_sin: Optional[torch.Tensor], row_pos: torch.Tensor, row_slot: torch.Tensor, page_table: torch.Tensor,
                q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                value_dim: int, rot_dims: int, eps: float, write_cache: bool = True) -> None:
    """Between the fused projection (float32) and attention: biases, RMS norm of q and of k over all heads at once
    (when weights are given), rotation of the first ``rot_dims`` dimensions of each head (i paired with i + rot_dims/2),
    q into ``q_out`` and k, v into the rows' places in the paged cache."""
    _need(qkv, "qkv", torch.float32)
    _need(q_out, "q_out")
    _need(k_cache, "k_cache", q_out.dtype)
    _need(v_cache, "v_cache", q_out.dtype)
    _need(row_pos, "row_pos", torch.int32)
    _need(row_slot, "row_slot", torch.int32)
    _need(page_table, "page_table", torch.int32)
    rows = qkv.shape[0]
    nq, nk, nv = heads * head_dim, kv_heads * head_dim, kv_heads * value_dim
    if qkv.shape[1] != nq + nk + nv or tuple(q_out.shape) != (rows, nq):
        raise KernelError(f"qkv_prepare: qkv {tuple(qkv.shape)} or q_out {tuple(q_out.shape)} do not fit the head sizes")
    if tuple(k_cache.shape[1:]) != (kv_heads, PAGE, head_dim) or tuple(v_cache.shape) != (k_cache.shape[0], kv_heads, PAGE, value_dim):
        raise KernelError(f"qkv_prepare: cache is {tuple(k_cache.shape)} and {tuple(v_cache.shape)}")
    for t, name, n in ((bias, "bias", nq + nk + nv), (q_weight, "q_weight", nq), (k_weight, "k_weight", nk)):
        if t is not None:
            _need(t, name, torch.float32)
            if t.numel() != n:
                raise KernelError(f"qkv_prepare: {name} has {t.numel()} values, wanted {n}")
    if (q_weight is None) != (k_weight is None):
        raise KernelError("qkv_prepare: the norm needs both weights or none")
    n_positions = 0
    if cos_sin is not None and rot_dims > 0:
        _need(cos_sin, "cos_sin", torch.float32)
        if cos_sin.shape[1] != rot_dims // 2:
            raise KernelError(f"qkv_prepare: the rotary table has {cos_sin.shape[1]} pairs, {rot_dims} rotated dimensions want {rot_dims // 2}")
        n_positions = cos_sin.shape[0]
        _bounds("qkv_prepare: row_pos", row_pos, n_positions, rows)
    _bounds_paged("qkv_prepare", rows, row_pos, row_slot, page_table, k_cache.shape[0])
    _call(_fn("bc_qkv_prepare_" + _suffix(q_out.dtype)), _ptr(qkv), _ptr(bias), _ptr(q_weight), _ptr(k_weight),
          _ptr(cos_sin if n_positions else None), _c_int(n_positions), _ptr(row_pos), _ptr(row_slot), _ptr(page_table),
          _c_int(page_table.shape[1]), _c_int(k_cache.shape[0]), _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _c_int(rows), _c_int(heads),
          _c_int(kv_heads), _c_int(head_dim), _c_int(value_dim), _c_int(rot_dims if n_positions else 0), _c_float(eps),
          _c_int(0 if q_weight is None else 1), _c_int(1 if write_cache else 0), _stream())


def qkv_prepare_heads(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], cos_sin: Optional[torch.Tensor],
                      row_pos: torch.Tensor, row_slot: torch.Tensor, page_table: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, heads: int, kv_heads: int, head_dim: int, value_dim: int, rot_dims: int, pairing: int, eps: float,
                      write_cache: bool = True) -> None:
    """Between the fused projection (float32) and attention for models that normalise every head by itself: an RMS norm of each
    head of q and of k over its ``head_dim`` values with weights of that many values shared by the heads (when given), rotation of
    the first ``rot_dims`` dimensions of each head (``pairing`` 0: i with i + rot_dims/2; 1: 2i with 2i + 1), q into ``q_out`` and
    k, v into the rows' places in the paged cache."""
    _need(qkv, "qkv", torch.float32)
    _need(q_out, "q_out")
    _need(k_cache, "k_cache", q_out.dtype)
    _need(v_cache, "v_cache", q_out.dtype)
    _need(row_pos, "row_pos", torch.int32)
    _need(row_slot, "row_slot", torch.int32)
    _need(page_table, "page_table", torch.int32)
    rows = qkv.shape[0]
    nq, nk, nv = heads * head_dim, kv_heads * head_dim, kv_heads * value_dim
    if qkv.shape[1] != nq + nk + nv or tuple(q_out.shape) != (rows, nq):
        raise KernelError(f"qkv_prepare_heads: qkv {tuple(qkv.shape)} or q_out {tuple(q_out.shape)} do not fit the head sizes")
    if tuple(k_cache.shape[1:]) != (kv_heads, PAGE, head_dim) or tuple(v_cache.shape) != (k_cache.shape[0], kv_heads, PAGE, value_dim):
        raise KernelError(f"qkv_prepare_heads: cache is {tuple(k_cache.shape)} and {tuple(v_cache.shape)}")
    if (q_weight is None) != (k_weight is None):
        raise KernelError("qkv_prepare_heads: the norm needs both weights or none")
    for t, name in ((q_weight, "q_weight"), (k_weight, "k_weight")):
        if t is not None:
            _need(t, name, torch.float32)
            if t.numel() != head_dim:
                raise KernelError(f"qkv_prepare_heads: {name} has {t.numel()} values, a head has {head_dim}")
    n_positions = 0
    if cos_sin is not None and rot_dims > 0:
        _need(cos_sin, "cos_sin", torch.float32)
        if cos_sin.shape[1] != rot_dims // 2:
            raise KernelError(f"qkv_prepare_heads: the rotary table has {cos_sin.shape[1]} pairs, {rot_dims} rotated dimensions want {rot_dims // 2}")
        n_positions = cos_sin.shape[0]
        _bounds("qkv_prepare_heads: row_pos", row_pos, n_positions, rows)
    _bounds_paged("qkv_prepare_heads", rows, row_pos, row_slot, page_table, k_cache.shape[0])
    _call(_fn("bc_qkv_prepare_heads_" + _suffix(q_out.dtype)), _ptr(qkv), _ptr(q_weight), _ptr(k_weight), _ptr(cos_sin if n_positions else None),
          _c_int(n_positions), _ptr(row_pos), _ptr(row_slot), _ptr(page_table), _c_int(page_table.shape[1]), _c_int(k_cache.shape[0]),
          _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _c_int(rows), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(value_dim),
          _c_int(rot_dims if n_positions else 0), _c_int(pairing), _c_float(eps), _c_int(0 if q_weight is None else 1),
          _c_int(1 if write_cache else 0), _stream())


# ----------------------------------------------------------- recurrences with a decaying outer-product state

def linear_scan(q: torch.Tensor, q_at: int, q_rep: int, k: torch.Tensor, k_at: int, k_rep: int, v: torch.Tensor, v_at: int,
                decay: torch.Tensor, decay_at: int, vector_decay: bool, kscale: Optional[torch.Tensor], kscale_at: int,
                skip: Optional[torch.Tensor], out_scale: float, state: torch.Tensor, seq_rows: torch.Tensor, seq_slot: torch.Tensor,
                out: torch.Tensor, seqs: int, heads: int, key_dim: int, value_dim: int, write_state: bool = True) -> None:
    """S_t = diag(a_t) S_(t-1) + (c_t k_t) v_t^T, o_t = out_scale * S_t^T q_t + skip * v_t for every head over every sequence's rows
    in time order, all float32.  q, k, v, decay and kscale are [rows, anything] tensors read from column ``*_at`` on: q and k hold
    ``key_dim`` values for each group of ``*_rep`` heads, v ``value_dim`` a head, decay ``key_dim`` a head (``vector_decay``) or one,
    kscale one a head (None: 1).  ``state`` [slots, heads, value_dim, key_dim] (value channel by value channel), ``out`` [rows, heads * value_dim]."""
    for t, name in ((q, "q"), (k, "k"), (v, "v"), (decay, "decay"), (state, "state"), (out, "out")):
        _need(t, name, torch.float32)
    _need(seq_rows, "seq_rows", torch.int32)
    _need(seq_slot, "seq_slot", torch.int32)
    H, N, P = heads, key_dim, value_dim
    rows = out.shape[0]
    if tuple(state.shape[1:]) != (H, P, N) or out.shape[1] != H * P or H % q_rep or H % k_rep:
        raise KernelError(f"linear_scan: state {tuple(state.shape)} or out {tuple(out.shape)} do not fit {H} heads of {N} x {P}")
    for t, at, width, name in ((q, q_at, H // q_rep * N, "q"), (k, k_at, H // k_rep * N, "k"), (v, v_at, H * P, "v"),
                               (decay, decay_at, H * N if vector_decay else H, "decay")):
        if t.dim() != 2 or t.shape[0] < rows or at < 0 or at + width > t.shape[1]:
            raise KernelError(f"linear_scan: {name} {tuple(t.shape)} has no {width} columns from {at} on for {rows} rows")
    if kscale is not None:
        _need(kscale, "kscale", torch.float32)
        if kscale.dim() != 2 or kscale.shape[0] < rows or kscale_at + H > kscale.shape[1]:
            raise KernelError(f"linear_scan: kscale {tuple(kscale.shape)} has no {H} columns from {kscale_at} on")
    if skip is not None:
        _need(skip, "skip", torch.float32)
        if skip.numel() != H:
            raise KernelError(f"linear_scan: skip has {skip.numel()} values for {H} heads")
    _bounds("linear_scan: seq_slot", seq_slot, state.shape[0], seqs, lowest=-1)
    _bounds("linear_scan: seq_rows", seq_rows, rows + 1, seqs + 1)

    def at(t, col):
        return _c_void_p(t.data_ptr() + 4 * col)

    _call(_fn("bc_linear_scan"), at(q, q_at), _c_int(q.shape[1]), _c_int(q_rep), at(k, k_at), _c_int(k.shape[1]), _c_int(k_rep), at(v, v_at),
          _c_int(v.shape[1]), at(decay, decay_at), _c_int(decay.shape[1]), _c_int(1 if vector_decay else 0),
          _c_void_p(0) if kscale is None else at(kscale, kscale_at), _c_int(0 if kscale is None else kscale.shape[1]), _ptr(skip),
          _c_float(out_scale), _ptr(state), _ptr(seq_rows), _ptr(seq_slot), _ptr(out), _c_int(seqs), _c_int(H), _c_int(N), _c_int(P),
          _c_int(state.shape[0]), _c_int(1 if write_state else 0), _stream())


SSD_MAX_TAPS = 9


def ssd_prepare(proj: torch.Tensor, conv_at: int, dt_at: int, weight_t: torch.Tensor, bias: Optional[torch.Tensor], dt_bias: torch.Tensor,
                a_log: torch.Tensor, tail: torch.Tensor, seq_rows: torch.Tensor, seq_slot: torch.Tensor, xbc: torch.Tensor, dtda: torch.Tensor,
                seqs: int, max_new: int, write_tail: bool = True) -> None:
    """xbc = silu(bias + causal convolution over time of proj's columns conv_at ..), channel by channel, with ``weight_t`` [taps, C]
    (the last tap is the current token's) and every slot's last taps - 1 inputs in ``tail`` [slots, taps - 1, C], brought up to date;
    dtda[r] = (softplus(dt + dt_bias), exp(-exp(a_log) * that)) for the H step sizes at proj's columns dt_at ...  All float32."""
    for t, name in ((proj, "proj"), (weight_t, "weight_t"), (dt_bias, "dt_bias"), (a_log, "a_log"), (tail, "tail"), (xbc, "xbc"), (dtda, "dtda")):
        _need(t, name, torch.float32)
    _need(seq_rows, "seq_rows", torch.int32)
    _need(seq_slot, "seq_slot", torch.int32)
    taps, C = weight_t.shape
    H = dt_bias.numel()
    rows = proj.shape[0]
    if a_log.numel() != H or tuple(xbc.shape) != (rows, C) or tuple(dtda.shape) != (rows, 2 * H) or conv_at + C > proj.shape[1] or dt_at + H > proj.shape[1]:
        raise KernelError(f"ssd_prepare: proj {tuple(proj.shape)}, xbc {tuple(xbc.shape)}, dtda {tuple(dtda.shape)} do not fit {C} channels and {H} heads")
    if tuple(tail.shape[1:]) != (max(taps - 1, 1), C) or not 1 <= taps <= SSD_MAX_TAPS:
        raise KernelError(f"ssd_prepare: tail {tuple(tail.shape)} does not fit {taps} taps of {C} channels (at most {SSD_MAX_TAPS} taps)")
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != C:
            raise KernelError(f"ssd_prepare: bias has {bias.numel()} values for {C} channels")
    _bounds("ssd_prepare: seq_slot", seq_slot, tail.shape[0], seqs, lowest=-1)
    _bounds("ssd_prepare: seq_rows", seq_rows, rows + 1, seqs + 1)
    _call(_fn("bc_ssd_prepare"), _ptr(proj), _c_int(proj.shape[1]), _c_int(conv_at), _c_int(dt_at), _ptr(weight_t), _ptr(bias), _ptr(dt_bias),
          _ptr(a_log), _ptr(tail), _ptr(seq_rows), _ptr(seq_slot), _ptr(xbc), _ptr(dtda), _c_int(seqs), _c_int(max_new), _c_int(C), _c_int(H),
          _c_int(taps), _c_int(tail.shape[0]), _c_int(1 if write_tail else 0), _stream())


def gla_decay(proj: torch.Tensor, inner_at: int, w2t: torch.Tensor, bias: torch.Tensor, decay: torch.Tensor, tau: float) -> None:
    """decay = sigmoid(z)^(1/tau) with z = inner @ w2t + bias, inner being proj's columns inner_at .. inner_at + rank; float32."""
    for t, name in ((proj, "proj"), (w2t, "w2t"), (bias, "bias"), (decay, "decay")):
        _need(t, name, torch.float32)
    rank, W = w2t.shape
    rows = proj.shape[0]
    if bias.numel() != W or tuple(decay.shape) != (rows, W) or inner_at + rank > proj.shape[1]:
        raise KernelError(f"gla_decay: proj {tuple(proj.shape)}, w2t {tuple(w2t.shape)}, decay {tuple(decay.shape)} do not fit")
    _call(_fn("bc_gla_decay"), _ptr(proj), _c_int(proj.shape[1]), _c_int(inner_at), _ptr(w2t), _ptr(bias), _ptr(decay), _c_int(rows), _c_int(W),
          _c_int(rank), _c_float(tau), _stream())


def gated_norm(y: torch.Tensor, gate: torch.Tensor, gate_at: int, weight: torch.Tensor, out: torch.Tensor, parts: int, eps: float,
               gate_first: bool, factor: float = 1.0, row_slot: Optional[torch.Tensor] = None) -> None:
    """Every row of y [rows, W] (float32) in ``parts`` equal parts, each divided by its own root mean square and multiplied by
    ``weight`` (as wide as the row, or as a part and then shared by the parts); silu of the gate (columns gate_at .. of ``gate``,
    float32) multiplies before the norm (``gate_first``) or after it; ``factor`` multiplies the result.  With ``row_slot``, rows whose
    slot is negative are not read and give zeros."""
    _need(y, "y", torch.float32)
    _need(gate, "gate", torch.float32)
    _need(weight, "weight", torch.float32)
    _need(out, "out")
    rows, W = y.shape
    if out.shape != y.shape or gate.shape[0] < rows or gate_at + W > gate.shape[1] or W % parts or weight.numel() not in (W, W // parts):
        raise KernelError(f"gated_norm: y {tuple(y.shape)}, gate {tuple(gate.shape)}, weight {weight.numel()}, {parts} parts do not fit")
    if row_slot is not None:
        _need(row_slot, "row_slot", torch.int32)
        if row_slot.numel() < rows:
            raise KernelError("gated_norm: fewer slots than rows")
    _call(_fn("bc_gated_norm_" + _suffix(out.dtype)), _ptr(y), _c_void_p(gate.data_ptr() + 4 * gate_at), _c_int(gate.shape[1]), _ptr(weight),
          _c_int(weight.numel()), _ptr(row_slot), _ptr(out), _c_int(rows), _c_int(W), _c_int(parts), _c_float(eps), _c_int(1 if gate_first else 0),
          _c_float(factor), _stream())


# ---------------------------------------------------------------------- attention whose heads talk

TALK_MAX_HEADS, TALK_MAX_DIM = 64, 256


def talk_prepare(proj: torch.Tensor, gate_at: int, bias: Optional[torch.Tensor], cos_sin: Optional[torch.Tensor], row_pos: torch.Tensor,
                 row_slot: torch.Tensor, page_table: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 gate: torch.Tensor, heads: int, kv_heads: int, head_dim: int, rot: int, eps: float, write_cache: bool = True) -> None:
    """From the fused projection proj [rows, P] float32 = [q | k | .. gate at ``gate_at`` ..]: q and k plus ``bias`` [(heads + kv_heads)
    head_dim], the first ``rot`` dimensions of every head rotated by the row's position (pairs (i, i + rot / 2)), every head divided by
    its root mean square; q into ``q_out`` [rows, heads * head_dim], k into ``k_cache`` and the key as projected (with its bias,
    neither rotated nor normed) into ``v_cache`` [pages, kv_heads, 64, head_dim] at the row's position; gate = sigmoid, float32
    [rows, heads * head_dim].  Rows whose slot is negative write no cache."""
    _need(proj, "proj", torch.float32)
    _need(q_out, "q_out")
    _need(k_cache, "k_cache", q_out.dtype)
    _need(v_cache, "v_cache", q_out.dtype)
    _need(gate, "gate", torch.float32)
    _need(page_table, "page_table", torch.int32)
    rows, P = proj.shape
    if tuple(q_out.shape) != (rows, heads * head_dim) or gate.shape != q_out.shape or tuple(k_cache.shape[1:]) != (kv_heads, PAGE, head_dim) \
            or v_cache.shape != k_cache.shape:
        raise KernelError(f"talk_prepare: q {tuple(q_out.shape)}, gate {tuple(gate.shape)}, cache {tuple(k_cache.shape)} and {tuple(v_cache.shape)} do not fit")
    if bias is not None:
        _need(bias, "bias", torch.float32)
        if bias.numel() != (heads + kv_heads) * head_dim:
            raise KernelError(f"talk_prepare: {bias.numel()} biases for {(heads + kv_heads) * head_dim} values")
    if rot > 0:
        _need(cos_sin, "cos_sin", torch.float32)
        if tuple(cos_sin.shape[1:]) != (rot // 2, 2):
            raise KernelError(f"talk_prepare: the rotary table is {tuple(cos_sin.shape)}, {rot} dimensions turn")
    _bounds_paged("talk_prepare", rows, row_pos, row_slot, page_table, k_cache.shape[0])
    _call(_fn("bc_talk_prepare_" + _suffix(q_out.dtype)), _ptr(proj), _c_int(rows), _c_int(P), _c_int(gate_at), _ptr(bias), _ptr(cos_sin if rot > 0 else None),
          _c_int(cos_sin.shape[0] if rot > 0 else 0), _ptr(row_pos), _ptr(row_slot), _ptr(page_table), _c_int(page_table.shape[1]), _c_int(k_cache.shape[0]),
          _ptr(q_out), _ptr(k_cache), _ptr(v_cache), _ptr(gate), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(rot), _c_float(eps),
          _c_int(1 if write_cache else 0), _stream())


def _talk_check(who: str, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, gate: torch.Tensor, temp: torch.Tensor, talk: torch.Tensor,
                out: torch.Tensor, heads: int, kv_heads: int, head_dim: int) -> None:
    _need(q, "q")
    _need(k_cache, "k_cache", q.dtype)
    _need(v_cache, "v_cache", q.dtype)
    _need(out, "out", q.dtype)
    for t, name in ((gate, "gate"), (temp, "temp"), (talk, "talk")):
        _need(t, name, torch.float32)
    rows = q.shape[0]
    if tuple(q.shape) != (rows, heads * head_dim) or out.shape != q.shape or gate.shape != q.shape or temp.numel() != heads \
            or talk.numel() != heads * heads or tuple(k_cache.shape[1:]) != (kv_heads, PAGE, head_dim) or v_cache.shape != k_cache.shape:
        raise KernelError(f"{who}: q {tuple(q.shape)}, gate {tuple(gate.shape)}, temp {temp.numel()}, talk {tuple(talk.shape)}, "
                          f"cache {tuple(k_cache.shape)} do not fit {heads} heads on {kv_heads} of {head_dim}")


def talk_rows(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor, row_pos: torch.Tensor, row_slot: torch.Tensor,
              gate: torch.Tensor, temp: torch.Tensor, talk: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int, head_dim: int, window: int,
              keep_first: int, scale: float, cap: float) -> None:
    """Attention whose heads' scores are mixed before the softmax, one block a row: raw score of head m = q_m . k * scale * temp[m],
    bounded by cap * tanh(. / cap) if ``cap`` > 0; head h's score = sum_m talk[h, m] raw_m; a row at position i sees j <= i with
    i - j < window or j < keep_first (window 0: all); out = gate * softmax-weighted sum of v.  Rows whose slot is negative give zeros."""
    _talk_check("talk_rows", q, k_cache, v_cache, gate, temp, talk, out, heads, kv_heads, head_dim)
    _need(page_table, "page_table", torch.int32)
    rows = q.shape[0]
    _bounds_paged("talk_rows", rows, row_pos, row_slot, page_table, k_cache.shape[0])
    _call(_fn("bc_talk_rows_" + _suffix(q.dtype)), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(page_table), _ptr(row_pos), _ptr(row_slot), _ptr(gate),
          _ptr(temp), _ptr(talk), _ptr(out), _c_int(rows), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page_table.shape[1]),
          _c_int(k_cache.shape[0]), _c_int(window), _c_int(keep_first), _c_float(scale), _c_float(cap), _stream())


def talk_tiles_accepts(heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tile kernel for prompts takes these sizes (bf16; up to 16 heads of a multiple of 16 up to 128, or up to 32 heads of
    up to 64, and a tile of all kv heads' keys and values that fits shared memory).  Otherwise talk_rows serves."""
    return dtype == torch.bfloat16 and bool(_fn("bc_talk_tiles_accepts")(_c_int(heads), _c_int(kv_heads), _c_int(head_dim)))


def talk_tiles(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor, seq_rows: torch.Tensor, seq_slot: torch.Tensor,
               seq_start: torch.Tensor, gate: torch.Tensor, temp: torch.Tensor, talk: torch.Tensor, out: torch.Tensor, seqs: int, max_new: int,
               heads: int, kv_heads: int, head_dim: int, window: int, keep_first: int, scale: float, cap: float, splits: int = 1,
               row_slot: Optional[torch.Tensor] = None) -> None:
    """What talk_rows computes, for bf16 on mma.sync tiles: a block owns sixteen rows of one sequence and all heads, so that
    every head can mix its score out of all heads' raw scores; sequence s brings rows seq_rows[s] .. seq_rows[s + 1] and held
    seq_start[s] positions before.  ``splits`` > 1 (steps of few rows a sequence) shares the positions a block would walk out over
    that many blocks and merges their parts in a second kernel, in the order of the splits; ``row_slot`` then marks padding rows."""
    _talk_check("talk_tiles", q, k_cache, v_cache, gate, temp, talk, out, heads, kv_heads, head_dim)
    _need(q, "q", torch.bfloat16)
    for t, name in ((page_table, "page_table"), (seq_rows, "seq_rows"), (seq_slot, "seq_slot"), (seq_start, "seq_start")):
        _need(t, name, torch.int32)
    if seq_rows.numel() < seqs + 1 or seq_slot.numel() < seqs or seq_start.numel() < seqs:
        raise KernelError("talk_tiles: fewer sequence entries than sequences")
    _bounds("talk_tiles: seq_slot", seq_slot, page_table.shape[0], seqs, lowest=-1)
    _bounds("talk_tiles: seq_rows", seq_rows, out.shape[0] + 1, seqs + 1)
    _bounds("talk_tiles: page_table", page_table, k_cache.shape[0], lowest=-1)
    scratch = None
    if splits > 1:
        _need(row_slot, "row_slot", torch.int32)
        scratch, _ = _decode_workspace(q.device, q.shape[0] * heads * splits * (head_dim + 2), 1)
    _call(_fn("bc_talk_tiles_bf16"), _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(page_table), _ptr(seq_rows), _ptr(seq_slot), _ptr(seq_start), _ptr(gate),
          _ptr(temp), _ptr(talk), _ptr(out), _c_int(seqs), _c_int(max_new), _c_int(heads), _c_int(kv_heads), _c_int(head_dim), _c_int(page_table.shape[1]),
          _c_int(k_cache.shape[0]), _c_int(window), _c_int(keep_first), _c_float(scale), _c_float(cap), _ptr(scratch), _c_int(splits),
          _ptr(row_slot if splits > 1 else None), _c_int(q.shape[0]), _stream())


def talk_tiles_splits(seqs: int, heads: int, reach: int, window: int, keep_first: int) -> int:
    """Splits of the positions a row sees (tiles of 32) for steps of few rows a sequence, so that the blocks fill the machine ONCE (a
    block takes most of a multiprocessor's shared memory, and more than sixteen heads take two or four blocks a sequence): never
    more than there are tiles (``reach``: a bound on the positions any row reaches; a window bounds them further)."""
    tiles = -(-max(reach, 1) // 32)
    if window > 0:
        tiles = min(tiles, -(-keep_first // 32) + (window + 30) // 32 + 1)
    blocks = max(seqs, 1) * (1 if heads <= 16 else 2 if heads <= 32 else 4)
    return max(1, min(tiles, sm_count() // blocks, 64))


# ------------------------------------------------------------------------------ routed experts

def moe_route(h: torch.Tensor, router: torch.Tensor, row_slot: Optional[torch.Tensor], logits: torch.Tensor, choice: torch.Tensor,
              weight: torch.Tensor, softmax: bool = False, renorm: bool = False, factor: float = 1.0) -> None:
    """choice [rows, top] (int32), weight [rows, top] (float32): every row's ``top`` experts by score, the lower index winning a tie.
    Scores are sigmoid(router @ h) (or a softmax over the experts), computed in float32; weights are the chosen scores, divided by
    their sum with ``renorm``, then times ``factor``.  Rows whose slot is negative choose nothing (-1).  ``logits`` [rows, experts] float32 receives router @ h."""
    _need(h, "h")
    _need(router, "router", torch.float32)
    _need(logits, "logits", torch.float32)
    _need(choice, "choice", torch.int32)
    _need(weight, "weight", torch.float32)
    rows, K = h.shape
    E, top = router.shape[0], choice.shape[1]
    if router.shape[1] != K or tuple(choice.shape) != (rows, top) or weight.shape != choice.shape or tuple(logits.shape) != (rows, E):
        raise KernelError(f"moe_route: h {tuple(h.shape)}, router {tuple(router.shape)}, choice {tuple(choice.shape)} do not fit")
    if row_slot is not None:
        _need(row_slot, "row_slot", torch.int32)
    _call(_fn("bc_moe_route_" + _suffix(h.dtype)), _ptr(h), _ptr(router), _ptr(row_slot), _ptr(logits), _ptr(choice), _ptr(weight), _c_int(rows), _c_int(E),
          _c_int(K), _c_int(top), _c_int(1 if softmax else 0), _c_int(1 if renorm else 0), _c_float(factor), _stream())


def moe_simt_tile_rows() -> int:
    """Sorted rows a tile of the CUDA-core expert product takes."""
    return int(_fn("bc_moe_simt_tile_rows")())


def moe_max_tiles(pairs: int, experts: int, tile_rows: Optional[int] = None) -> int:
    return int(_fn("bc_moe_max_tiles")(_c_int(pairs), _c_int(experts), _c_int(moe_simt_tile_rows() if tile_rows is None else tile_rows)))


def moe_plan(choice: torch.Tensor, experts: int, counts: torch.Tensor, offsets: torch.Tensor, table: torch.Tensor, perm: torch.Tensor,
             place: torch.Tensor, tile_rows: Optional[int] = None) -> None:
    """Sorts the (row, choice) pairs by expert: perm[j] names the pair at sorted place j, place[pair] its place; ``table`` lists tiles
    of at most ``tile_rows`` sorted rows (default: what the CUDA-core product takes) that lie in one expert ([0]: how many; then
    expert, first place, rows for each)."""
    tile_rows = moe_simt_tile_rows() if tile_rows is None else int(tile_rows)
    for t, name in ((choice, "choice"), (counts, "counts"), (offsets, "offsets"), (table, "table"), (perm, "perm"), (place, "place")):
        _need(t, name, torch.int32)
    pairs = choice.numel()
    if counts.numel() < experts or offsets.numel() < experts + 1 or table.numel() < 1 + 3 * moe_max_tiles(pairs, experts, tile_rows) or perm.numel() < pairs \
            or place.numel() < pairs:
        raise KernelError("moe_plan: a buffer is too small")
    _call(_fn("bc_moe_plan"), _ptr(choice), _c_int(pairs), _c_int(experts), _c_int(tile_rows), _ptr(counts), _ptr(offsets), _ptr(table), _ptr(perm),
          _ptr(place), _stream())


def moe_gather(x: torch.Tensor, perm: torch.Tensor, offsets: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, experts: int, top: int,
               weight_on_input: bool) -> None:
    """out[j] = x[row of the pair at sorted place j], times the pair's weight with ``weight_on_input``; places past the pairs that
    chose an expert are cleared."""
    _need(x, "x")
    _need(out, "out", x.dtype)
    _need(perm, "perm", torch.int32)
    _need(offsets, "offsets", torch.int32)
    _need(weight, "weight", torch.float32)
    pairs, K = out.shape
    if x.shape[1] != K or perm.numel() < pairs or offsets.numel() < experts + 1 or weight.numel() < pairs:
        raise KernelError(f"moe_gather: x {tuple(x.shape)}, out {tuple(out.shape)} do not fit")
    _call(_fn("bc_moe_gather_" + _suffix(x.dtype)), _ptr(x), _ptr(perm), _ptr(offsets), _ptr(weight), _ptr(out), _c_int(pairs), _c_int(experts),
          _c_int(K), _c_int(top), _c_int(1 if weight_on_input else 0), _stream())


GROUPED_TILE_ROWS = (16, 32, 64, 128, 256)


def gemm_tc_grouped_accepts(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core product over groups of rows takes these operands (bf16, K a multiple of 8, 16-byte aligned)."""
    return x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def gemm_tc_grouped(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, table: torch.Tensor, gated: bool, tile_rows: int, max_tiles: int,
                    relu2: bool = False) -> None:
    """Rows of x [rows, K] sorted by the matrix they meet, times that matrix of w [matrices, N, K] (``gated``: [matrices, 2 N, K],
    gate rows then up rows, and out = silu(gate) * up in bf16; ``relu2``: out = max(sum, 0)^2 in bf16; else out float32 [rows, N]),
    on the tcgen05 tensor cores.  ``table``
    ([0]: tiles; then matrix, first row, rows a tile of at most ``tile_rows``) comes from ``moe_plan`` with the same ``tile_rows``."""
    _need(x, "x", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    if gated and relu2:
        raise KernelError("gemm_tc_grouped: a gated product has its own activation")
    _need(out, "out", torch.bfloat16 if gated or relu2 else torch.float32)
    _need(table, "table", torch.int32)
    rows, K = x.shape
    matrices, n_w, kw = w.shape
    N = n_w // 2 if gated else n_w
    if kw != K or tuple(out.shape) != (rows, N) or tile_rows not in GROUPED_TILE_ROWS or table.numel() < 1 + 3 * max_tiles:
        raise KernelError(f"gemm_tc_grouped: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, tiles of {tile_rows} do not fit")
    _call(_fn("bc_gemm_tc_grouped_bf16"), _ptr(x), _ptr(w), _ptr(out), _ptr(table), _c_int(rows), _c_int(matrices), _c_int(N), _c_int(K),
          _c_int(1 if gated else 2 if relu2 else 0), _c_int(tile_rows), _c_int(max_tiles), _stream())


def moe_product(gated: bool, x: torch.Tensor, w: torch.Tensor, table: torch.Tensor, perm: torch.Tensor, weight: torch.Tensor, out: torch.Tensor,
                top: int, weight_on_input: bool = False) -> None:
    """The experts' products over rows sorted by expert.  ``gated``: x [rows, K], w [E, 2 N, K] (gate rows, then up rows), out
    [pairs, N] = silu(s g) * (s u) in x's type, s the pair's weight (1 unless ``weight_on_input``).  Else: x [pairs, K] in sorted
    order, w [E, N, K], out [pairs, N] float32."""
    _need(x, "x")
    _need(w, "w", x.dtype)
    _need(out, "out", x.dtype if gated else torch.float32)
    E, n_w, K = w.shape
    N = n_w // 2 if gated else n_w
    pairs = out.shape[0]
    if x.shape[1] != K or out.shape[1] != N or (not gated and x.shape[0] != pairs) or perm.numel() < pairs:
        raise KernelError(f"moe_product: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
    _call(_fn("bc_moe_product_" + _suffix(x.dtype)), _c_int(1 if gated else 0), _ptr(x), _ptr(w), _ptr(table), _ptr(perm), _ptr(weight), _ptr(out),
          _c_int(pairs), _c_int(E), _c_int(N), _c_int(K), _c_int(top), _c_int(1 if weight_on_input else 0), _stream())


def moe_combine(y: torch.Tensor, choice: torch.Tensor, place: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor,
                weight_on_output: bool = False) -> None:
    """residual[r] += the sum over row r's choices, in their order, of y[place of the pair] (times the pair's weight with ``weight_on_output``)."""
    _need(y, "y", torch.float32)
    _need(residual, "residual", torch.float32)
    rows, top = choice.shape
    if y.shape[1] != residual.shape[1] or residual.shape[0] < rows:
        raise KernelError(f"moe_combine: y {tuple(y.shape)} and residual {tuple(residual.shape)} do not fit")
    _call(_fn("bc_moe_combine"), _ptr(y), _ptr(choice), _ptr(place), _ptr(weight), _ptr(residual), _c_int(rows), _c_int(residual.shape[1]),
          _c_int(top), _c_int(1 if weight_on_output else 0), _stream())


# ---------------------------------------------------------------------------- latent attention

def latent_prepare(proj: torch.Tensor, q_rank: int, kv_at: int, kv_rank: int, rot: int, gate_at: int, heads: int, q_weight: torch.Tensor,
                   kv_weight: Optional[torch.Tensor], cos_sin: Optional[torch.Tensor], row_pos: torch.Tensor, row_slot: torch.Tensor,
                   page_table: Optional[torch.Tensor], c_pages: Optional[torch.Tensor], r_pages: Optional[torch.Tensor], cq: torch.Tensor,
                   gate: torch.Tensor, eps: float, write_cache: bool = True) -> None:
    """From a row of the fused down projection ``proj`` (float32: ``q_rank`` values at 0; at ``kv_at`` ``kv_rank`` values and
    ``rot`` more, unless ``kv_at`` < 0; ``heads`` values at ``gate_at``): cq = RMS norm of the first part times ``q_weight`` in cq's
    type; the RMS norm of the second part times ``kv_weight`` and the ``rot`` values rotated by the row's position (pairs
    (i, i + rot / 2), ``cos_sin`` [positions, rot / 2, 2]) into the row's place of ``c_pages`` [pages, 1, 64, kv_rank] and ``r_pages``
    [pages, 1, 64, rot]; gate = sigmoid of the third part (float32).  Rows whose slot is negative write nothing into the cache."""
    _need(proj, "proj", torch.float32)
    _need(cq, "cq")
    _need(gate, "gate", torch.float32)
    _need(q_weight, "q_weight", torch.float32)
    rows, P = proj.shape
    writes = kv_at >= 0 and write_cache
    if tuple(cq.shape) != (rows, q_rank) or tuple(gate.shape) != (rows, heads) or q_weight.numel() != q_rank:
        raise KernelError(f"latent_prepare: proj {tuple(proj.shape)}, cq {tuple(cq.shape)}, gate {tuple(gate.shape)} do not fit")
    n_pages = max_pages = 0
    if writes:
        _need(c_pages, "c_pages", cq.dtype)
        _need(kv_weight, "kv_weight", torch.float32)
        _need(page_table, "page_table", torch.int32)
        n_pages, max_pages = c_pages.shape[0], page_table.shape[1]
        if c_pages.shape[-1] != kv_rank or c_pages.shape[-2] != PAGE or kv_weight.numel() != kv_rank:
            raise KernelError(f"latent_prepare: pages of {tuple(c_pages.shape)} do not hold latents of {kv_rank}")
        if rot > 0:
            _need(r_pages, "r_pages", cq.dtype)
            _need(cos_sin, "cos_sin", torch.float32)
            if r_pages.shape[-1] != rot or r_pages.shape[0] != n_pages or cos_sin.shape[1] * 2 != rot:
                raise KernelError(f"latent_prepare: rotated keys of {rot} do not fit pages {tuple(r_pages.shape)} or a table of {tuple(cos_sin.shape)}")
        _bounds_paged("latent_prepare", rows, row_pos, row_slot, page_table, n_pages)
        if rot > 0:
            _bounds("latent_prepare: row_pos", row_pos, cos_sin.shape[0], rows)
    _call(_fn("bc_latent_prepare_" + _suffix(cq.dtype)), _ptr(proj), _c_int(rows), _c_int(P), _c_int(q_rank), _c_int(kv_at), _c_int(kv_rank), _c_int(rot),
          _c_int(gate_at), _c_int(heads), _ptr(q_weight), _ptr(kv_weight), _ptr(cos_sin), _c_int(0 if cos_sin is None else cos_sin.shape[0]), _ptr(row_pos),
          _ptr(row_slot), _ptr(page_table), _c_int(max_pages), _c_int(n_pages), _ptr(c_pages if writes else None), _ptr(r_pages if writes else None),
          _ptr(cq), _ptr(gate), _c_float(eps), _c_int(1 if writes else 0), _stream())


def latent_query(q: torch.Tensor, w_uk: torch.Tensor, cos_sin: Optional[torch.Tensor], row_pos: torch.Tensor, out: torch.Tensor, heads: int, dim: int,
                 rot: int, kv_rank: int) -> None:
    """out[r, n] = [Wuk_n^T q_n | rot(qr_n)]: q float32 [rows, heads * (dim + rot)], head by head ``dim`` plain values then ``rot``
    rotated ones; ``w_uk`` [heads * dim, kv_rank]; out [rows, heads, kv_rank + rot] in w_uk's type."""
    _need(q, "q", torch.float32)
    _need(w_uk, "w_uk")
    _need(out, "out", w_uk.dtype)
    rows = q.shape[0]
    if q.shape[1] != heads * (dim + rot) or tuple(w_uk.shape) != (heads * dim, kv_rank) or out.numel() != rows * heads * (kv_rank + rot):
        raise KernelError(f"latent_query: q {tuple(q.shape)}, w_uk {tuple(w_uk.shape)}, out {tuple(out.shape)} do not fit")
    if rot > 0:
        _need(cos_sin, "cos_sin", torch.float32)
        _bounds("latent_query: row_pos", row_pos, cos_sin.shape[0], rows)
    _call(_fn("bc_latent_query_" + _suffix(w_uk.dtype)), _ptr(q), _ptr(w_uk), _ptr(cos_sin if rot > 0 else None),
          _c_int(cos_sin.shape[0] if rot > 0 else 0), _ptr(row_pos), _ptr(out), _c_int(rows), _c_int(heads), _c_int(dim), _c_int(rot), _c_int(kv_rank), _stream())


LATENT_MAX_RANK, LATENT_MAX_ROT = 512, 128


def latent_rows(a: torch.Tensor, c_pages: torch.Tensor, r_pages: Optional[torch.Tensor], page_table: torch.Tensor, row_pos: torch.Tensor,
                row_slot: torch.Tensor, out: torch.Tensor, heads: int, kv_rank: int, rot: int, window: int, scale: float,
                sink: Optional[torch.Tensor] = None) -> None:
    """Attention over cached latents, one warp a (row, head): a [rows, heads, kv_rank + rot] are the absorbed queries, every head
    reads the same ``c_pages`` [pages, 1, 64, kv_rank] (keys and values at once) and ``r_pages`` [pages, 1, 64, rot];
    out [rows, heads, kv_rank] = sum_j softmax_j((a_c . c_j + a_r . r_j) * scale) c_j over the positions j the row sees
    (``window`` > 0: the last ``window`` ones, itself included).  ``sink`` float32 [heads]: every head's softmax has one more term
    e^sink in its denominator, without a key or a value.  Rows whose slot is negative give zeros."""
    _need(a, "a")
    _sink_values(sink, heads, "latent_rows")
    _need(c_pages, "c_pages", a.dtype)
    _need(out, "out", a.dtype)
    _need(page_table, "page_table", torch.int32)
    rows = a.shape[0]
    if a.numel() != rows * heads * (kv_rank + rot) or out.numel() != rows * heads * kv_rank or c_pages.shape[-1] != kv_rank:
        raise KernelError(f"latent_rows: a {tuple(a.shape)}, out {tuple(out.shape)}, pages {tuple(c_pages.shape)} do not fit")
    if rot > 0:
        _need(r_pages, "r_pages", a.dtype)
    _bounds_paged("latent_rows", rows, row_pos, row_slot, page_table, c_pages.shape[0])
    _call(_fn("bc_latent_rows_" + _suffix(a.dtype)), _ptr(a), _ptr(c_pages), _ptr(r_pages if rot > 0 else None), _ptr(page_table), _ptr(row_pos),
          _ptr(row_slot), _ptr(out), _c_int(rows), _c_int(heads), _c_int(kv_rank), _c_int(rot), _c_int(page_table.shape[1]), _c_int(c_pages.shape[0]),
          _c_int(window), _c_float(scale), _ptr(sink), _stream())


def latent_values(ctx: torch.Tensor, w_uv: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, heads: int, kv_rank: int, value_dim: int) -> None:
    """out[r, n] = gate[r, n] * Wuv_n ctx[r, n]: ctx [rows, heads, kv_rank], ``w_uv`` [heads * value_dim, kv_rank], gate float32
    [rows, heads], out [rows, heads * value_dim] in ctx's type."""
    _need(ctx, "ctx")
    _need(w_uv, "w_uv", ctx.dtype)
    _need(gate, "gate", torch.float32)
    _need(out, "out", ctx.dtype)
    rows = out.shape[0]
    if ctx.numel() != rows * heads * kv_rank or tuple(w_uv.shape) != (heads * value_dim, kv_rank) or out.shape[1] != heads * value_dim \
            or gate.numel() != rows * heads:
        raise KernelError(f"latent_values: ctx {tuple(ctx.shape)}, w_uv {tuple(w_uv.shape)}, out {tuple(out.shape)} do not fit")
    _call(_fn("bc_latent_values_" + _suffix(ctx.dtype)), _ptr(ctx), _ptr(w_uv), _ptr(gate), _ptr(out), _c_int(rows), _c_int(heads), _c_int(kv_rank),
          _c_int(value_dim), _stream())


def latent_decode_accepts(heads: int, kv_rank: int, rot: int, dtype: torch.dtype) -> bool:
    """Whether the split kernel for single rows takes these sizes (bf16; a latent in multiples of 8 up to 512, a rotated part in
    multiples of 8 up to 128).  Otherwise latent_rows serves."""
    return dtype == torch.bfloat16 and bool(_fn("bc_latent_decode_accepts")(_c_int(heads), _c_int(kv_rank), _c_int(rot)))


def latent_decode_splits(rows: int, heads: int, reach: int, window: int, kv_rank: int = 0, rot: int = 0) -> int:
    """Splits of the cached positions so that rows * (groups of sixteen heads) * splits blocks fill the machine ONCE: as many
    blocks as are resident together (two stages of a page's rows [c | r] a block, so wide latents leave one block a
    multiprocessor and a second wave would double the time), never more than a row can see pages (``reach``: a bound on the
    positions any row reaches)."""
    tiles = -(-max(reach, 1) // PAGE)
    if window > 0:
        tiles = min(tiles, (window + PAGE - 2) // PAGE + 1)
    blocks = max(1, rows * (-(-heads // 16)))
    resident = 2
    if kv_rank > 0:
        shared = (16 + 2 * PAGE) * (-(-(kv_rank + rot) // 16) * 16 + 8) * 2 + 16 * 72 * 2 + 512
        resident = max(1, min(8, (227 * 1024) // (shared + 1024)))
    return max(1, min(resident * sm_count() // blocks, tiles, 64))


def latent_decode(a: torch.Tensor, c_pages: torch.Tensor, r_pages: Optional[torch.Tensor], page_table: torch.Tensor, row_pos: torch.Tensor,
                  row_slot: torch.Tensor, out: torch.Tensor, heads: int, kv_rank: int, rot: int, window: int, scale: float,
                  splits: Optional[int] = None, reach: Optional[int] = None, sink: Optional[torch.Tensor] = None) -> None:
    """What latent_rows computes, for bf16 and few rows: a block takes (row, sixteen heads, split of the cached positions), the
    heads sharing every read of the cache on mma.sync tiles; several splits are merged in their order by a second kernel.
    The result does not depend on ``reach``, only the number of splits chosen does."""
    for t, name in ((a, "a"), (c_pages, "c_pages"), (out, "out")):
        _need(t, name, torch.bfloat16)
    _need(page_table, "page_table", torch.int32)
    _sink_values(sink, heads, "latent_decode")
    rows = a.shape[0]
    if a.numel() != rows * heads * (kv_rank + rot) or out.numel() != rows * heads * kv_rank or c_pages.shape[-1] != kv_rank:
        raise KernelError(f"latent_decode: a {tuple(a.shape)}, out {tuple(out.shape)}, pages {tuple(c_pages.shape)} do not fit")
    if rot > 0:
        _need(r_pages, "r_pages", torch.bfloat16)
    if splits is None:
        splits = latent_decode_splits(rows, heads, page_table.shape[1] * PAGE if reach is None else reach, window, kv_rank, rot)
    scratch = None
    if splits > 1:
        floats = rows * (-(-heads // 16)) * splits * (32 + 16 * (-(-kv_rank // 16) * 16))     # a split leaves 16 maxima, 16 sums, 16 rows
        scratch, _ = _decode_workspace(a.device, floats, 1)
    _bounds_paged("latent_decode", rows, row_pos, row_slot, page_table, c_pages.shape[0])
    _call(_fn("bc_latent_decode_bf16"), _ptr(a), _ptr(c_pages), _ptr(r_pages if rot > 0 else None), _ptr(page_table), _ptr(row_pos), _ptr(row_slot),
          _ptr(out), _ptr(scratch), _c_int(rows), _c_int(heads), _c_int(kv_rank), _c_int(rot), _c_int(page_table.shape[1]), _c_int(c_pages.shape[0]),
          _c_int(window), _c_float(scale), _c_int(splits), _ptr(sink), _stream())


def latent_heads(q: torch.Tensor, cos_sin: Optional[torch.Tensor], row_pos: torch.Tensor, out: torch.Tensor, heads: int, dim: int, rot: int) -> None:
    """out [rows, heads, padded] (bf16) = every head's query as it meets expanded keys: ``dim`` plain values, ``rot`` values rotated
    by the row's position (pairs (i, i + rot / 2)), zeros up to the padded width.  q float32 [rows, heads * (dim + rot)]."""
    _need(q, "q", torch.float32)
    _need(out, "out", torch.bfloat16)
    rows = q.shape[0]
    padded = out.numel() // max(rows * heads, 1)
    if q.shape[1] != heads * (dim + rot) or out.numel() != rows * heads * padded or padded < dim + rot:
        raise KernelError(f"latent_heads: q {tuple(q.shape)} and out {tuple(out.shape)} do not fit")
    if rot > 0:
        _need(cos_sin, "cos_sin", torch.float32)
        _bounds("latent_heads: row_pos", row_pos, cos_sin.shape[0], rows)
    _call(_fn("bc_latent_heads_bf16"), _ptr(q), _ptr(cos_sin if rot > 0 else None), _c_int(cos_sin.shape[0] if rot > 0 else 0), _ptr(row_pos), _ptr(out),
          _c_int(rows), _c_int(heads), _c_int(dim), _c_int(rot), _c_int(padded), _stream())


def latent_gather(c_pages: torch.Tensor, r_pages: Optional[torch.Tensor], page_table: torch.Tensor, pg_slot: torch.Tensor, pg_pos: torch.Tensor,
                  pg_last: torch.Tensor, ctx_c: torch.Tensor, ctx_r: Optional[torch.Tensor], pages: int) -> None:
    """Copies, for scratch page p, the cache's rows of slot ``pg_slot[p]`` at positions ``pg_pos[p]`` .. + 63 (a multiple of 64)
    into ctx_c [pages * 64, kv_rank] and ctx_r [pages * 64, rot]; rows past position ``pg_last[p]`` and pages the cache does not
    hold become zeros."""
    _need(c_pages, "c_pages", torch.bfloat16)
    _need(ctx_c, "ctx_c", torch.bfloat16)
    for t, name in ((page_table, "page_table"), (pg_slot, "pg_slot"), (pg_pos, "pg_pos"), (pg_last, "pg_last")):
        _need(t, name, torch.int32)
    R = c_pages.shape[-1]
    rot = 0 if r_pages is None else r_pages.shape[-1]
    if ctx_c.numel() < pages * PAGE * R or (rot and (ctx_r is None or ctx_r.numel() < pages * PAGE * rot)) or min(pg_slot.numel(), pg_pos.numel(),
                                                                                                                 pg_last.numel()) < pages:
        raise KernelError("latent_gather: the outputs or the pages' lists are shorter than the pages")
    _bounds("latent_gather: pg_slot", pg_slot, page_table.shape[0], pages, lowest=-1)
    _call(_fn("bc_latent_gather_bf16"), _ptr(c_pages), _ptr(r_pages), _ptr(page_table), _ptr(pg_slot), _ptr(pg_pos), _ptr(pg_last), _ptr(ctx_c),
          _ptr(ctx_r if rot else None), _c_int(pages), _c_int(R), _c_int(rot), _c_int(page_table.shape[1]), _c_int(c_pages.shape[0]), _stream())


def latent_spread(kv: torch.Tensor, ctx_r: Optional[torch.Tensor], keys: torch.Tensor, values: torch.Tensor, heads: int, dim: int, value_dim: int,
                  rot: int) -> None:
    """kv [S, heads * dim + heads * value_dim] (every head's plain key part, then every head's values) and the shared rotated part
    ctx_r [S, rot] -> keys [S / 64, heads, 64, padded] = [key part | rotated part | zeros] and values [S / 64, heads, 64, padded]."""
    for t, name in ((kv, "kv"), (keys, "keys"), (values, "values")):
        _need(t, name, torch.bfloat16)
    S = kv.shape[0]
    if kv.shape[1] != heads * (dim + value_dim) or S % PAGE or tuple(keys.shape[:3]) != (S // PAGE, heads, PAGE) \
            or tuple(values.shape[:3]) != (S // PAGE, heads, PAGE) or keys.shape[3] < dim + rot or values.shape[3] < value_dim:
        raise KernelError(f"latent_spread: kv {tuple(kv.shape)}, keys {tuple(keys.shape)}, values {tuple(values.shape)} do not fit")
    if rot > 0:
        _need(ctx_r, "ctx_r", torch.bfloat16)
    _call(_fn("bc_latent_spread_bf16"), _ptr(kv), _ptr(ctx_r if rot > 0 else None), _ptr(keys), _ptr(values), _c_int(S), _c_int(heads), _c_int(dim),
          _c_int(value_dim), _c_int(rot), _c_int(keys.shape[3]), _c_int(values.shape[3]), _stream())


def latent_gate(att: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, heads: int, value_dim: int) -> None:
    """out [rows, heads * value_dim] = att [rows, heads, padded][..., :value_dim] * gate [rows, heads] (float32)."""
    _need(att, "att", torch.bfloat16)
    _need(gate, "gate", torch.float32)
    _need(out, "out", torch.bfloat16)
    rows = out.shape[0]
    padded = att.numel() // max(rows * heads, 1)
    if out.shape[1] != heads * value_dim or att.numel() != rows * heads * padded or padded < value_dim or gate.numel() != rows * heads:
        raise KernelError(f"latent_gate: att {tuple(att.shape)}, gate {tuple(gate.shape)}, out {tuple(out.shape)} do not fit")
    _call(_fn("bc_latent_gate_bf16"), _ptr(att), _ptr(gate), _ptr(out), _c_int(rows), _c_int(heads), _c_int(value_dim), _c_int(padded), _stream())


def latent_expand_widths(heads: int, key_dim: int, value_dim: int, kv_rank: int, rot: int, dtype: torch.dtype):
    """(padded key width, padded value width) under which the prompt attention kernels take a latent mixer's expanded keys
    (``key_dim`` = plain + rotated values a head) and values, or None: bf16, latents and rotated parts in multiples of 8.
    Widths of 64 and 128 (values no wider than keys) run on the tcgen05 kernel; else equal widths in multiples of 16 up to 128
    on mma.sync tiles."""
    if dtype != torch.bfloat16 or kv_rank % 8 or rot % 8 or max(key_dim, value_dim) > 128:
        return None
    vp = 64 if value_dim <= 64 else 128
    kp = max(64 if key_dim <= 64 else 128, vp)
    if attention_prefill_tc_accepts(heads, heads, kp, value_dim=vp):
        return kp, vp
    w = -(-max(key_dim, value_dim) // 16) * 16
    return (w, w) if attention_tiles_accepts(heads, heads, w, w, dtype) else None


# ------------------------------------------------------------- norms after a sublayer, relu squared

def norm_add(y: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, eps: float) -> None:
    """residual[r] += y[r] * rsqrt(mean(y[r]^2) + eps) * weight for the rows of y; all float32."""
    _need(y, "y", torch.float32)
    _need(weight, "weight", torch.float32)
    _need(residual, "residual", torch.float32)
    rows, E = y.shape
    if residual.shape[0] < rows or residual.shape[1] != E or weight.numel() != E:
        raise KernelError(f"norm_add: y {tuple(y.shape)}, residual {tuple(residual.shape)}, weight {weight.numel()} do not fit")
    _call(_fn("bc_norm_add_f32"), _ptr(y), _ptr(weight), _ptr(residual), _c_int(rows), _c_int(E), _c_float(eps), _stream())


def norm_add_norm(y: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor, eps: float, next_weight: torch.Tensor, out: torch.Tensor,
                  next_eps: float) -> None:
    """norm_add, then out[r] = residual[r] * rsqrt(mean(residual[r]^2) + next_eps) * next_weight in out's type, and y = 0: what lies
    between the two sublayers of a block that norms before and after each, in one kernel.  y, residual and the weights float32."""
    _need(y, "y", torch.float32)
    _need(weight, "weight", torch.float32)
    _need(next_weight, "next_weight", torch.float32)
    _need(residual, "residual", torch.float32)
    _need(out, "out")
    rows, E = y.shape
    if residual.shape[0] < rows or residual.shape[1] != E or weight.numel() != E or next_weight.numel() != E or tuple(out.shape) != (rows, E):
        raise KernelError(f"norm_add_norm: y {tuple(y.shape)}, residual {tuple(residual.shape)}, out {tuple(out.shape)}, weights {weight.numel()} and "
                          f"{next_weight.numel()} do not fit")
    _call(_fn("bc_norm_add_norm_" + _suffix(out.dtype)), _ptr(y), _ptr(weight), _ptr(residual), _ptr(next_weight), _ptr(out), _c_int(rows), _c_int(E),
          _c_float(eps), _c_float(next_eps), _stream())


def relu2(z: torch.Tensor, out: torch.Tensor) -> None:
    """out = max(z, 0)^2: z float32, out of any type the kernels know, the same shape."""
    _need(z, "z", torch.float32)
    _need(out, "out")
    if out.shape != z.shape:
        raise KernelError(f"relu2: z {tuple(z.shape)} and out {tuple(out.shape)} differ")
    _call(_fn("bc_relu2_" + _suffix(out.dtype)), _ptr(z), _ptr(out), ctypes.c_longlong(z.numel()), _stream())


def glu_clipped(z: torch.Tensor, out: torch.Tensor, limit: float, alpha: float) -> None:
    """out[r, j] = g sigmoid(alpha g) (u + 1) with g = min(z[r, j], limit) and u = clamp(z[r, F + j], -limit, limit): z float32
    [rows, 2 F] (a gate/up product's sums), out [rows, F] of any type the kernels know."""
    _need(z, "z", torch.float32)
    _need(out, "out")
    rows, F = out.shape
    if tuple(z.shape) != (rows, 2 * F):
        raise KernelError(f"glu_clipped: z is {tuple(z.shape)}, wanted {(rows, 2 * F)}")
    _call(_fn("bc_glu_clipped_" + _suffix(out.dtype)), _ptr(z), _ptr(out), _c_int(rows), _c_int(F), _c_float(limit), _c_float(alpha), _stream())


def gated_add(h: torch.Tensor, g: torch.Tensor, y: torch.Tensor, residual: torch.Tensor) -> None:
    """residual[r] += sigmoid(g . h[r]) * y[r]: h [rows, K] and g [K] of one type, y and residual float32 [rows, E]."""
    _need(h, "h")
    _need(g, "g", h.dtype)
    _need(y, "y", torch.float32)
    _need(residual, "residual", torch.float32)
    rows, K = h.shape
    if g.numel() != K or y.shape[0] != rows or residual.shape[0] < rows or residual.shape[1] != y.shape[1]:
        raise KernelError(f"gated_add: h {tuple(h.shape)}, g {g.numel()}, y {tuple(y.shape)}, residual {tuple(residual.shape)} do not fit")
    _call(_fn("bc_gated_add_" + _suffix(h.dtype)), _ptr(h), _ptr(g), _ptr(y), _ptr(residual), _c_int(rows), _c_int(K), _c_int(y.shape[1]), _stream())


def moe_table_route(table: torch.Tensor, tokens: torch.Tensor, row_slot: Optional[torch.Tensor], choice: torch.Tensor, weight: torch.Tensor,
                    experts: int) -> None:
    """choice[r] = table[tokens[r]] ([vocabulary, top] int32), weight = 1 / top: the experts of a row are named by its token id.
    Rows whose slot is negative, and entries outside the experts, choose nothing (-1)."""
    _need(table, "table", torch.int32)
    _need(tokens, "tokens", torch.int32)
    _need(choice, "choice", torch.int32)
    _need(weight, "weight", torch.float32)
    rows, top = choice.shape
    if table.shape[1] != top or tokens.numel() < rows or weight.shape != choice.shape:
        raise KernelError(f"moe_table_route: table {tuple(table.shape)}, choice {tuple(choice.shape)} do not fit")
    _call(_fn("bc_moe_table_route"), _ptr(table), _ptr(tokens), _ptr(row_slot), _ptr(choice), _ptr(weight), _c_int(rows), _c_int(table.shape[0]),
          _c_int(experts), _c_int(top), _stream())


# ----------------------------------------------------------------------- the stream and the scores

def softcap(scores: torch.Tensor, cap: float) -> None:
    """scores <- cap * tanh(scores / cap), in place; float32."""
    _need(scores, "scores", torch.float32)
    _call(_fn("bc_softcap_f32"), _ptr(scores), ctypes.c_longlong(scores.numel()), _c_float(cap), _stream())


def scale_scores(scores: torch.Tensor, factor: float) -> None:
    """scores <- factor * scores, in place; float32."""
    _need(scores, "scores", torch.float32)
    _call(_fn("bc_scale_f32"), _ptr(scores), ctypes.c_longlong(scores.numel()), _c_float(factor), _stream())


def add_bias(x: torch.Tensor, b: torch.Tensor) -> None:
    """x[r] += b: x float32 [rows, E], b float32 [E] (the bias of a product whose epilogue adds into x)."""
    _need(x, "x", torch.float32)
    _need(b, "b", torch.float32)
    rows, E = x.shape
    if b.numel() != E:
        raise KernelError(f"add_bias: {b.numel()} biases for rows of {E}")
    _call(_fn("bc_add_bias_f32"), _ptr(x), _ptr(b), _c_int(rows), _c_int(E), _stream())


def reentry(x: torch.Tensor, x0: torch.Tensor, step: torch.Tensor, cat: torch.Tensor) -> None:
    """cat[r] = [x[r]; x0[r]] in cat's type, then x[r] <- step: the operand of the product that mixes the stream with the
    embedding's output, and the vector its epilogue adds onto."""
    _need(x, "x", torch.float32)
    _need(x0, "x0", torch.float32)
    _need(step, "step", torch.float32)
    _need(cat, "cat")
    rows, E = x.shape
    if x0.shape != x.shape or step.numel() != E or tuple(cat.shape) != (rows, 2 * E):
        raise KernelError(f"reentry: x {tuple(x.shape)}, x0 {tuple(x0.shape)}, step {step.numel()}, cat {tuple(cat.shape)} do not fit")
    _call(_fn("bc_reentry_" + _suffix(cat.dtype)), _ptr(x), _ptr(x0), _ptr(step), _ptr(cat), _c_int(rows), _c_int(E), _stream())


_decode_scratch = {}


def set_attention_decode_tma(on: bool) -> None:
    """Whether the decode attention fetches pages by TMA where the head size (64, 128) allows
    (the default) or by cp.async everywhere; both give the same bits.  For measurements and tests."""
    lib().bc_attention_decode_set_tma(_c_int(1 if on else 0))


def set_attention_decode_cluster16(on: bool) -> None:
    """Whether sixteen splits of the decode attention run as one thread-block cluster of
    sixteen where the device places one (the default) or as two clusters of eight whose sums
    go through scratch memory.  For measurements and tests."""
    lib().bc_attention_decode_set_cluster16(_c_int(1 if on else 0))


def attention_decode_accepts(heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the split decode kernel takes these sizes (bf16; at most 16 heads a kv head;
    head size a multiple of 16 up to 128).  Otherwise attention_rows serves."""
    return dtype == torch.bfloat16 and bool(_fn("bc_attention_decode_accepts")(_c_int(heads), _c_int(kv_heads), _c_int(head_dim)))


def attention_decode_splits(rows: int, kv_heads: int, max_pages: int) -> int:
    """Splits of the cached positions so that rows * kv_heads * splits blocks come close to,
    and stay within, one wave of two blocks on each SM; never more than a sequence
    can have pages.  Up to eight splits merge inside a thread-block cluster, which costs
    about 4 us less than the merge through scratch memory; so eight is the cap unless the
    batch is so small that eight leave most SMs idle and the sequences are long.  Then:
    sixteen as one cluster of sixteen, where all of these find an SM each (one sequence of
    eight kv heads, from 64 pages on: 13 against 18 us a launch at 8,000 positions); and
    beyond 192 pages (320 where sixteen serve) a multiple of eight: clusters of eight merge
    among themselves and only their sums go through scratch memory (32 against 59 us at
    32,000 positions)."""
    blocks = max(1, rows * kv_heads)
    sms = sm_count()
    fill = max(1, min(2 * sms // blocks, max_pages, 64))
    if fill <= 8 or blocks * 8 >= sms:
        # A power of two: clusters of 3, 5, 6 or 7 blocks place badly once the SMs fill up
        # (five sequences of eight kv heads: 20.7 us with 7 splits, 14.7 us with 4).
        return 1 << (min(fill, 8).bit_length() - 1)
    sixteen = blocks * 16 <= sms and fill >= 16
    if sixteen and 64 < max_pages <= 320:
        return 16
    if max_pages <= 192 or (sixteen and max_pages <= 64):
        return 8
    return fill // 8 * 8


def _decode_workspace(device: torch.device, floats: int, ints: int):
    """Scratch of the split decode kernel, one a device, grown outside of any capture and
    never freed (a captured graph keeps pointing at the buffer it saw)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    held = _decode_scratch.setdefault(key, [])
    for f, c in held:
        if f.numel() >= floats and c.numel() >= ints:
            return f, c
    if torch.cuda.is_current_stream_capturing():
        raise KernelError("attention_decode: scratch memory must exist before a graph is captured (run the step once eagerly)")
    f = torch.empty(max(floats, 1 << 20), dtype=torch.float32, device=device)
    c = torch.zeros(max(ints, 1 << 14), dtype=torch.int32, device=device)
    held.append((f, c))
    return f, c


def attention_decode(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor,
                     row_pos: torch.Tensor, row_slot: torch.Tensor, out: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                     window: int = 0, scale: Optional[float] = None, splits: Optional[int] = None, fuse: int = 0,
                     cos_sin: Optional[torch.Tensor] = None, pairing: int = 0, via_scratch: bool = False,
                     reach: Optional[int] = None, sink: bool = False, out_scale: float = 1.0) -> None:
    """Attention of one new row a sequence (bf16): the cached positions are split across
    blocks and the heads of a kv head share each read; results are merged in a fixed order.
    Two to eight splits form a thread-block cluster and merge through one another's shared
    memory; more (or ``via_scratch``) merge through scratch memory, with the same result.
    ``fuse`` 1 or 2: ``q`` is the fused projection as the product left it; q is rotated on
    the fly by ``cos_sin`` (None: no rotation), and with 2 the row's rotated key and its
    value are appended to the cache first (what rope_append would have done).  ``reach``:
    a bound on the positions any row reaches (else what the page table can hold); the
    number of splits is chosen by it, no result depends on it.  ``sink`` adds one to the softmax's
    denominator (a position of score 0 without a value), ``out_scale`` multiplies the result: both
    with the plain kernel (``fuse`` 0) only."""
    _need(q, "q", torch.bfloat16)
    _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16)
    _need(page_table, "page_table", torch.int32)
    _need(row_pos, "row_pos", torch.int32)
    _need(row_slot, "row_slot", torch.int32)
    _need(out, "out", torch.bfloat16)
    rows = out.shape[0]
    if out.shape[1] != heads * head_dim:
        raise KernelError(f"attention: out width {out.shape[1]} is not heads * head_dim")
    if tuple(k_cache.shape[1:]) != (kv_heads, PAGE, head_dim) or k_cache.shape != v_cache.shape:
        raise KernelError(f"attention: cache is {tuple(k_cache.shape)}, wanted [pages, {kv_heads}, {PAGE}, {head_dim}]")
    if scale is None:
        scale = 1.0 / float(head_dim) ** 0.5
    if splits is None:
        pages = page_table.shape[1]
        if reach is not None:
            pages = min(pages, -(-max(1, reach) // PAGE))
        if window > 0:
            pages = min(pages, -(-window // PAGE) + 1)
        splits = attention_decode_splits(rows, kv_heads, pages)
    scratch = counters = None
    if splits > 1:
        scratch, counters = _decode_workspace(q.device, rows * heads * splits * (head_dim + 2), rows * kv_heads)
    if cos_sin is not None:
        _need(cos_sin, "cos_sin", torch.float32)
        if tuple(cos_sin.shape[1:]) != (head_dim // 2, 2):
            raise KernelError(f"attention_decode: cos_sin is {tuple(cos_sin.shape)}, wanted [positions, {head_dim // 2}, 2]")
        if bounds_check and not torch.cuda.is_current_stream_capturing():
            _bounds("attention_decode: row_pos (against the rotary table)", row_pos.reshape(-1)[:rows][row_slot.reshape(-1)[:rows] >= 0], cos_sin.shape[0])
    _bounds_paged("attention_decode", rows, row_pos, row_slot, page_table, k_cache.shape[0])
    if sink or out_scale != 1.0:
        if fuse != 0:
            raise KernelError("attention_decode: a sink or a factor comes with the plain kernel (fuse 0)")
        _call(_fn("bc_attention_decode_sink_bf16"), _ptr(q), _c_int(q_stride), _ptr(k_cache), _ptr(v_cache), _ptr(page_table), _ptr(row_pos),
              _ptr(row_slot), _ptr(out), _ptr(scratch), _ptr(counters), _c_int(rows), _c_int(heads), _c_int(kv_heads), _c_int(head_dim),
              _c_int(page_table.shape[1]), _c_int(k_cache.shape[0]), _c_int(window), _c_float(scale), _c_int(splits),
              _c_int(4 if via_scratch else 0), _c_int(1 if sink else 0), _c_float(out_scale), _stream())
        return
    _call(_fn("bc_attention_decode_fused_bf16"), _ptr(q), _c_int(q_stride), _ptr(k_cache), _ptr(v_cache), _ptr(page_table), _ptr(row_pos),
          _ptr(row_slot), _ptr(out), _ptr(scratch), _ptr(counters), _c_int(rows), _c_int(heads), _c_int(kv_heads), _c_int(head_dim),
          _c_int(page_table.shape[1]), _c_int(k_cache.shape[0]), _c_int(window), _c_float(scale), _c_int(splits), _ptr(cos_sin),
          _c_int(pairing), _c_int(fuse + (4 if via_scratch else 0)), _stream())


def attention_prefill_accepts(heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tiled prompt kernel takes these sizes (bf16; at most 64 heads a kv head;
    head size a multiple of 16 up to 128).  Otherwise attention_rows serves."""
    return dtype == torch.bfloat16 and bool(_fn("bc_attention_prefill_accepts")(_c_int(heads), _c_int(kv_heads), _c_int(head_dim)))


def attention_tiles_accepts(heads: int, kv_heads: int, head_dim: int, value_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tiled kernel takes keys of ``head_dim`` with values of ``value_dim`` (bf16; equal widths in
    multiples of 16 up to 128, or keys of 32, 64, 128 with values of 16, 32, 64, 128)."""
    return dtype == torch.bfloat16 and bool(_fn("bc_attention_prefill_kv_accepts")(_c_int(heads), _c_int(kv_heads), _c_int(head_dim),
                                                                                  _c_int(value_dim)))


def attention_tiles(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor,
                    seq_rows: torch.Tensor, seq_slot: torch.Tensor, seq_start: torch.Tensor, out: torch.Tensor, seqs: int, max_new: int,
                    heads: int, kv_heads: int, head_dim: int, value_dim: int, window: int = 0, chunk: int = 0,
                    scale: Optional[float] = None, sink: bool = False, out_scale: float = 1.0) -> None:
    """Causal attention of every sequence's new rows (many, or one) against its cached positions on mma.sync
    tiles, bf16, with values of their own width, a sliding window and/or a chunk mask (``chunk`` > 0: a position
    sees only those of its own chunk of that many positions, counted from position 0).  ``sink`` adds one to the
    softmax's denominator (a position of score 0 without a value), or, given as a float32 tensor [heads], e^sink[head];
    ``out_scale`` multiplies the result."""
    for t, name in ((q, "q"), (k_cache, "k_cache"), (v_cache, "v_cache"), (out, "out")):
        _need(t, name, torch.bfloat16)
    if isinstance(sink, torch.Tensor):
        _sink_values(sink, heads, "attention_tiles")
    for t, name in ((page_table, "page_table"), (seq_rows, "seq_rows"), (seq_slot, "seq_slot"), (seq_start, "seq_start")):
        _need(t, name, torch.int32)
    if out.shape[1] != heads * value_dim:
        raise KernelError(f"attention: out width {out.shape[1]} is not heads * value_dim")
    if tuple(k_cache.shape[1:]) != (kv_heads, PAGE, head_dim) or tuple(v_cache.shape) != (k_cache.shape[0], kv_heads, PAGE, value_dim):
        raise KernelError(f"attention: cache is {tuple(k_cache.shape)} and {tuple(v_cache.shape)}")
    if scale is None:
        scale = 1.0 / float(head_dim) ** 0.5
    _bounds("attention_tiles: seq_slot", seq_slot, page_table.shape[0], seqs, lowest=-1)
    _bounds("attention_tiles: seq_rows", seq_rows, out.shape[0] + 1, seqs + 1)
    _bounds("attention_tiles: page_table", page_table, k_cache.shape[0], lowest=-1)
    _call(_fn("bc_attention_prefill_sink_bf16"), _ptr(q), _c_int(q_stride), _ptr(k_cache), _ptr(v_cache), _ptr(page_table), _ptr(seq_rows),
          _ptr(seq_slot), _ptr(seq_start), _ptr(out), _c_int(seqs), _c_int(max_new), _c_int(heads), _c_int(kv_heads), _c_int(head_dim),
          _c_int(value_dim), _c_int(page_table.shape[1]), _c_int(k_cache.shape[0]), _c_int(window), _c_int(chunk), _c_float(scale),
          _c_int(0 if sink is None or sink is False else 1), _ptr(sink if isinstance(sink, torch.Tensor) else None), _c_float(out_scale), _stream())


def attention_prefill_tc_accepts(heads: int, kv_heads: int, head_dim: int, q: Optional[torch.Tensor] = None, q_stride: int = 0,
                                 value_dim: Optional[int] = None) -> bool:
    """Whether the tcgen05 prompt kernel takes these sizes (head size 64 or 128, at most 128
    heads a kv head, values of 64 or 128 and no wider than the keys) and, if given, this q
    (16-byte aligned, row stride a multiple of 8)."""
    if not _fn("bc_attention_prefill_tc_accepts_kv")(_c_int(heads), _c_int(kv_heads), _c_int(head_dim),
                                                     _c_int(head_dim if value_dim is None else value_dim)):
        return False
    return q is None or (q.data_ptr() % 16 == 0 and q_stride % 8 == 0)


def attention_prefill(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor,
                      seq_rows: torch.Tensor, seq_slot: torch.Tensor, seq_start: torch.Tensor, out: torch.Tensor, seqs: int, max_new: int,
                      heads: int, kv_heads: int, head_dim: int, window: int = 0, scale: Optional[float] = None,
                      use_tc: Optional[bool] = None, chunk: int = 0, value_dim: Optional[int] = None, sink: bool = False,
                      out_scale: float = 1.0) -> None:
    """Causal attention of every sequence's new rows against its cached positions (which
    include the new rows' own keys and values), bf16.  Head sizes 64 and 128 run on the
    tcgen05 tensor cores, 128 query rows a block (scores and output accumulate in TMEM);
    other head sizes on mma.sync tiles, 64 rows a block.  ``use_tc`` forces one or the other.
    ``chunk`` > 0: a position sees only those of its own chunk of that many positions, counted from position 0.
    ``value_dim`` (default ``head_dim``): the width of a head's values, in v_cache and in out.
    ``sink`` adds one to the softmax's denominator (a position of score 0 without a value), or, given as a float32 tensor [heads],
    e^sink[head]; ``out_scale`` multiplies the result."""
    value_dim = head_dim if value_dim is None else int(value_dim)
    if isinstance(sink, torch.Tensor):
        _sink_values(sink, heads, "attention_prefill")
    _need(q, "q", torch.bfloat16)
    _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16)
    _need(page_table, "page_table", torch.int32)
    _need(seq_rows, "seq_rows", torch.int32)
    _need(seq_slot, "seq_slot", torch.int32)
    _need(seq_start, "seq_start", torch.int32)
    _need(out, "out", torch.bfloat16)
    if out.shape[1] != heads * value_dim:
        raise KernelError(f"attention: out width {out.shape[1]} is not heads * value_dim")
    if tuple(k_cache.shape[1:]) != (kv_heads, PAGE, head_dim) or tuple(v_cache.shape) != (k_cache.shape[0], kv_heads, PAGE, value_dim):
        raise KernelError(f"attention: cache is {tuple(k_cache.shape)} and {tuple(v_cache.shape)}, wanted [pages, {kv_heads}, {PAGE}, {head_dim}] "
                          f"and values {value_dim} wide")
    if seq_rows.numel() < seqs + 1 or seq_slot.numel() < seqs or seq_start.numel() < seqs:
        raise KernelError("attention_prefill: fewer sequence entries than sequences")
    if scale is None:
        scale = 1.0 / float(head_dim) ** 0.5
    if bounds_check and not torch.cuda.is_current_stream_capturing():
        _bounds("attention_prefill: seq_slot", seq_slot, page_table.shape[0], seqs, lowest=-1)
        _bounds("attention_prefill: seq_rows", seq_rows, out.shape[0] + 1, seqs + 1)
        live = seq_slot.reshape(-1)[:seqs] >= 0
        ends = (seq_start.reshape(-1)[:seqs] + seq_rows.reshape(-1)[1:seqs + 1] - seq_rows.reshape(-1)[:seqs])[live]
        _bounds("attention_prefill: a sequence's last position + 1", ends, page_table.shape[1] * PAGE + 1)
        _bounds("attention_prefill: page_table", page_table, k_cache.shape[0], lowest=-1)
    if use_tc is None:
        use_tc = attention_prefill_tc_accepts(heads, kv_heads, head_dim, q, q_stride, value_dim)
    if use_tc:
        _call(_fn("bc_attention_prefill_tc_sink_bf16"), _ptr(q), _c_int(q_stride), _c_int(out.shape[0]), _ptr(k_cache), _ptr(v_cache), _ptr(page_table),
              _ptr(seq_rows), _ptr(seq_slot), _ptr(seq_start), _ptr(out), _c_int(seqs), _c_int(max_new), _c_int(heads), _c_int(kv_heads),
              _c_int(head_dim), _c_int(value_dim), _c_int(page_table.shape[1]), _c_int(k_cache.shape[0]), _c_int(window), _c_int(chunk),
              _c_float(scale), _c_int(0 if sink is None or sink is False else 1), _ptr(sink if isinstance(sink, torch.Tensor) else None),
              _c_float(out_scale), _stream())
        return
    if chunk > 0 or value_dim != head_dim or (sink is not None and sink is not False) or out_scale != 1.0:
        attention_tiles(q, q_stride, k_cache, v_cache, page_table, seq_rows, seq_slot, seq_start, out, seqs, max_new, heads, kv_heads, head_dim,
                        value_dim, window=window, chunk=chunk, scale=scale, sink=sink, out_scale=out_scale)
        return
    _call(_fn("bc_attention_prefill_bf16"), _ptr(q), _c_int(q_stride), _ptr(k_cache), _ptr(v_cache), _ptr(page_table), _ptr(seq_rows),
          _ptr(seq_slot), _ptr(seq_start), _ptr(out), _c_int(seqs), _c_int(max_new), _c_int(heads), _c_int(kv_heads), _c_int(head_dim),
          _c_int(page_table.shape[1]), _c_int(k_cache.shape[0]), _c_int(window), _c_float(scale), _stream())


# ---------------------------------------------------------------------------------- sampling

def argmax(scores: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the first largest score of row r."""
    _need(scores, "scores", torch.float32)
    _need(out, "out", torch.int32)
    rows, V = scores.shape
    _call(_fn("bc_argmax"), _ptr(scores), _c_int(rows), _c_int(V), _ptr(out), _stream())


def set_sample_blocks_per_row(n: int) -> None:
    """Blocks that share a row of the sampler: 0 lets the launcher choose (eight while all
    rows still run at once, fewer for more rows), 1, 2, 4 or 8 force it.  For measurements and tests."""
    lib().bc_sample_set_blocks_per_row(_c_int(int(n)))


def sample(scores: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, seed: torch.Tensor, step: torch.Tensor,
           out: torch.Tensor) -> None:
    """One draw a row: greedy where temperature <= 0, else temperature / nucleus sampling
    with the draw keyed by (seed, step).  seed is int64 (its bits are the 64-bit seed)."""
    _need(scores, "scores", torch.float32)
    _need(temperature, "temperature", torch.float32)
    _need(top_p, "top_p", torch.float32)
    _need(seed, "seed", torch.int64)
    _need(step, "step", torch.int32)
    _need(out, "out", torch.int32)
    rows, V = scores.shape
    for name, t in (("temperature", temperature), ("top_p", top_p), ("seed", seed), ("step", step), ("out", out)):
        if t.numel() < rows:
            raise KernelError(f"sample: {name} has fewer entries than rows")
    _call(_fn("bc_sample"), _ptr(scores), _c_int(rows), _c_int(V), _ptr(temperature), _ptr(top_p), _ptr(seed), _ptr(step), _ptr(out), _stream())
