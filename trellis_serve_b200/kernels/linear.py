"""Dense EXL3 linear on B200: the function surface of the reference's kernel backend
(cuda/src/sglang_exl3/kernels/marlin.py of 0xSero/trellis-serve) over libexl3_b200's C ABI.

Same names, argument meaning and error behaviour as the reference module: `probe`, `supports`, `prepare`, `run`
for the serving path and the building blocks `had_in_group`, `had_out_into`, `supports_matrix`, `prepare_matrix`,
`unprepare_matrix`, `gemm_rotated`, `gemm_rotated_group`, `linear`, `linear_group` for parity tools; plus
`reconstruct`, which stands in for the third-party decoder the reference calls
(cuda/src/sglang_exl3/kernels/reference.py:71-80).  What differs is what the reference could not serve: every
integer K in 2..8 and all three codebooks (its own kernels: K in {3,4,5,6}, codebooks mcg / mul1 only,
marlin.py:51-62).

Activations may be fp16 or bf16; the product always runs on fp16 values.  bf16 is converted exactly as torch's
`.to(float16)` / `.to(bfloat16)` would, so `run(x_bf16) == run(x_bf16.half()).bfloat16()` bit for bit
(marlin.py:9-12).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib
from .base import BackendStatus

MAX_ROWS = 64            # rows the per-device workspace is sized for at load time (marlin.py:24-27)
_workspace: dict[int, torch.Tensor] = {}
_tc_workspace: dict[int, torch.Tensor] = {}


def _dtype_code(t: torch.Tensor, allow_f32: bool = False) -> int:
    if t.dtype == torch.float16:
        return _lib.F16
    if t.dtype == torch.bfloat16:
        return _lib.BF16
    if allow_f32 and t.dtype == torch.float32:
        return _lib.F32
    raise TypeError(f"activations must be fp16 or bf16, got {t.dtype}")


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t: torch.Tensor | None):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _bits(trellis_or_words) -> int:
    words = trellis_or_words if isinstance(trellis_or_words, int) else trellis_or_words.shape[2]
    return words // 16


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor: the EXL3 kernels have no CPU path")


def workspace_bytes(rows: int, k: int, n_total: int, shards: int) -> int:
    return int(_lib.load().exl3_linear_workspace_bytes(min(rows, 16), k, n_total, shards))


def reserve_workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-filled, reused per-device scratch (activation fragments, split-k partial sums, counters).  Sized at load
    time so the run path never allocates and CUDA graphs see a fixed address."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    cur = _workspace.get(idx)
    if cur is None or cur.numel() < nbytes:
        cur = _workspace[idx] = torch.zeros(nbytes, dtype=torch.uint8, device=torch.device("cuda", idx))
    return cur


def probe() -> BackendStatus:
    try:
        lib = _lib.load()
    except (ImportError, OSError) as e:
        return BackendStatus(False, detail=str(e))
    return BackendStatus(True, version=str(lib.exl3_version()))


def supports(trellis: list[torch.Tensor], out_widths: list[int], codebooks: list[int]) -> tuple[bool, str]:
    if len({t.shape[2] for t in trellis}) != 1 or trellis[0].shape[2] % 16 or not 2 <= trellis[0].shape[2] // 16 <= 8:
        return False, "one bitrate per group, integer K in 2..8"
    if any((t.shape[0] * 16) % 128 or (t.shape[1] * 16) % 128 for t in trellis):
        return False, "k, n not multiples of 128"
    if len(set(codebooks)) != 1 or codebooks[0] not in (0, 1, 2):
        return False, "one codebook per group: 3inst, mcg or mul1"
    if any(w != t.shape[1] * 16 for w, t in zip(out_widths, trellis)):
        return False, "padded output columns"
    if len({t.shape[0] for t in trellis}) != 1:
        return False, "different input widths"
    if len(trellis) > 4:
        return False, "more than 4 matrices in one group"
    return True, ""


def supports_matrix(trellis: torch.Tensor) -> tuple[bool, str]:
    k, n = trellis.shape[0] * 16, trellis.shape[1] * 16
    if trellis.shape[2] % 16 or not 2 <= trellis.shape[2] // 16 <= 8:
        return False, f"K = {trellis.shape[2] / 16:g} (integer K in 2..8 only)"
    if k % 128 or n % 128:
        return False, f"k, n = {k}, {n} not multiples of 128"
    return True, ""


def prepare_matrix(trellis: torch.Tensor) -> torch.Tensor:
    """int16 (k/16, n/16, 16K) -> resident int32 (n/128, k/128, 8, 2, K, 32): the same bits, lane-major."""
    _require_cuda(trellis, "trellis")
    ok, why = supports_matrix(trellis)
    if not ok:
        raise RuntimeError(f"cannot prepare this matrix: {why}")
    lib = _lib.load()
    _lib.init_device(trellis.device.index)
    t = trellis.contiguous()
    kt, nt, words = t.shape
    K = words // 16
    packed = torch.empty((nt // 8, kt // 8, 8, 2, K, 32), dtype=torch.int32, device=t.device)
    with torch.cuda.device(t.device):
        _lib.check(lib.exl3_repack(_ptr(t), kt * 16, nt * 16, K, _ptr(packed), _stream(t.device)), "exl3_repack")
    return packed


def unprepare_matrix(packed: torch.Tensor) -> torch.Tensor:
    """Exact inverse of `prepare_matrix`."""
    lib = _lib.load()
    nb, kg, _, _, K, _ = packed.shape
    p = packed.contiguous()
    out = torch.empty((kg * 8, nb * 8, 16 * K), dtype=torch.int16, device=p.device)
    with torch.cuda.device(p.device):
        _lib.check(lib.exl3_unpack(_ptr(p), kg * 128, nb * 128, K, _ptr(out), _stream(p.device)), "exl3_unpack")
    return out


def prepare(trellis: list[torch.Tensor], suh: list[torch.Tensor], svh: list[torch.Tensor]):
    """-> (packed int32 [n_total/128, k/128, 8, 2, K, 32], suh_cat [shards, k], svh_cat [n_total], shard_ends)."""
    b = torch.cat([prepare_matrix(t) for t in trellis], dim=0).contiguous()
    ends, total = [], 0
    for t in trellis[:-1]:
        total += t.shape[1] * 16
        ends.append(total)
    k = trellis[0].shape[0] * 16
    n_total = sum(t.shape[1] * 16 for t in trellis)
    reserve_workspace(b.device, workspace_bytes(MAX_ROWS, k, n_total, len(trellis)))
    suh_cat, svh_cat = torch.stack(suh).contiguous(), torch.cat(svh).contiguous()
    # The run path starts fetching the resident weights and sign vectors while the kernel ahead of it is still running
    # (programmatic dependent launch), so they must be complete before the first `run` is enqueued: load time pays for that.
    torch.cuda.current_stream(b.device).synchronize()
    return b, suh_cat, svh_cat, ends


def _geometry(packed: torch.Tensor) -> tuple[int, int, int]:
    nb, kg, _, _, K, _ = packed.shape
    return kg * 128, nb * 128, K


def _own_or_given(workspace: torch.Tensor | None, device: torch.device, need: int, table: dict) -> torch.Tensor:
    """The caller's scratch when one is handed in (it must be large enough: nothing is allocated on its behalf), else the
    per-device one of this module, grown if needed."""
    if workspace is not None:
        if workspace.numel() * workspace.element_size() < need:
            raise RuntimeError(f"workspace holds {workspace.numel() * workspace.element_size()} bytes, this call needs {need}")
        return workspace
    idx = device.index if device.index is not None else torch.cuda.current_device()
    cur = table.get(idx)
    if cur is None or cur.numel() < need:
        cur = table[idx] = torch.zeros(need, dtype=torch.uint8, device=torch.device("cuda", idx))
    return cur


def run(x: torch.Tensor, b: torch.Tensor, suh_cat: torch.Tensor, svh_cat: torch.Tensor, shard_ends: list[int],
        codebook: int, out: torch.Tensor | None = None, exchange=None, workspace: torch.Tensor | None = None) -> torch.Tensor:
    """x fp16 | bf16 [rows, k] contiguous -> y (same dtype) [rows, n_total].  Only y is allocated (unless `out`).
    `workspace`: caller-owned zero-filled scratch of at least `workspace_bytes(...)` (default: this module's own).
    An fp32 `out` receives the unrounded accumulators (accuracy measurements).  `exchange` (a
    `runtime.allreduce.PeerAllReduce`): the matrix is a row-parallel shard and y is summed over the ranks inside the
    kernel, the same bits as `exchange(run(...))`."""
    _require_cuda(x, "x")
    lib = _lib.load()
    _lib.init_device(x.device.index if x.device.index is not None else torch.cuda.current_device())
    rows, kx = x.shape
    k, n_total, K = _geometry(b)
    if kx != k:
        raise RuntimeError(f"x has width {kx}, the packed weights expect {k}")
    shards = len(shard_ends) + 1
    y = out if out is not None else torch.empty((rows, n_total), dtype=x.dtype, device=x.device)
    if rows == 0:
        return y
    ws = _own_or_given(workspace, x.device, workspace_bytes(rows, k, n_total, shards), _workspace)
    with torch.cuda.device(x.device):
        if exchange is not None and exchange.world > 1:
            _lib.check(lib.exl3_linear_allreduce(_ptr(x), _dtype_code(x), _ptr(b), K, codebook, _ptr(suh_cat), _ptr(svh_cat),
                                                 _lib.int_array(shard_ends), shards, rows, k, n_total, _ptr(y), _dtype_code(y),
                                                 _ptr(ws), ws.numel(), exchange.peer_regions, exchange.rank, exchange.world,
                                                 exchange.max_elems, _ptr(exchange.state), _stream(x.device)),
                       "exl3_linear_allreduce")
        else:
            _lib.check(lib.exl3_linear(_ptr(x), _dtype_code(x), _ptr(b), K, codebook, _ptr(suh_cat), _ptr(svh_cat),
                                       _lib.int_array(shard_ends), shards, rows, k, n_total, _ptr(y), _dtype_code(y, True),
                                       _ptr(ws), ws.numel(), _stream(x.device)), "exl3_linear")
    return y


def tc_workspace_bytes(rows: int, k: int, n_total: int, shards: int) -> int:
    return int(_lib.load().exl3_gemm_tc_workspace_bytes(rows, k, n_total, shards))


def run_tc(x: torch.Tensor, b: torch.Tensor, suh_cat: torch.Tensor, svh_cat: torch.Tensor, shard_ends: list[int],
           codebook: int, out: torch.Tensor | None = None, workspace: torch.Tensor | None = None) -> torch.Tensor:
    """Many-row version of `run` on the tcgen05 tensor cores: weights decoded once per 512 rows into the MMA operand.
    `workspace`: caller-owned scratch of at least `tc_workspace_bytes(...)` whose first 256 bytes are zero."""
    _require_cuda(x, "x")
    lib = _lib.load()
    _lib.init_device(x.device.index if x.device.index is not None else torch.cuda.current_device())
    rows, kx = x.shape
    k, n_total, K = _geometry(b)
    if kx != k:
        raise RuntimeError(f"x has width {kx}, the packed weights expect {k}")
    shards = len(shard_ends) + 1
    y = out if out is not None else torch.empty((rows, n_total), dtype=x.dtype, device=x.device)
    if rows == 0:
        return y
    ws = _own_or_given(workspace, x.device, tc_workspace_bytes(rows, k, n_total, shards), _tc_workspace)
    with torch.cuda.device(x.device):
        _lib.check(lib.exl3_linear_tc(_ptr(x), _dtype_code(x), _ptr(b), K, codebook, _ptr(suh_cat), _ptr(svh_cat),
                                      _lib.int_array(shard_ends), shards, rows, k, n_total, _ptr(y), _dtype_code(y), _ptr(ws),
                                      ws.numel(), _stream(x.device)), "exl3_linear_tc")
    return y


# ---------------------------------------------------------------------------------------------------------------
# Decode step: the kernel ahead of a linear writes the linear's rotated input (residual / normalisation / activation fused
# with the input rotation), the linear runs from those fragments.  All four share one workspace in stream order.

def _step_workspace(device: torch.device, rows: int, k: int, shards: int, workspace: torch.Tensor) -> torch.Tensor:
    """The chain's workspace is the caller's (zero-filled once, `workspace_bytes` of the largest group): the fragments one
    call leaves there are what the next call reads, so no call may swap the buffer for a larger one on its own."""
    if workspace is None:
        raise RuntimeError("the decode-step calls share one caller-owned workspace: pass it to every call of the chain")
    _lib.init_device(device.index if device.index is not None else torch.cuda.current_device())
    return _own_or_given(workspace, device, workspace_bytes(rows, k, 128, shards), _workspace)


def rotate_fragments(x: torch.Tensor, suh_cat: torch.Tensor, codebook: int, workspace: torch.Tensor) -> None:
    """Fragments of Had128(fp16(x) * suh[s]) for every matrix s of the following group, into the workspace."""
    _require_cuda(x, "x")
    rows, k = x.shape
    shards = suh_cat.numel() // k
    ws = _step_workspace(x.device, rows, k, shards, workspace)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().exl3_rotate_fragments(_ptr(x), _dtype_code(x), _ptr(suh_cat), shards, rows, k, codebook, _ptr(ws),
                                                     ws.numel(), _stream(x.device)), "exl3_rotate_fragments")


def rmsnorm_rotate(x: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor, eps: float, suh_cat: torch.Tensor,
                   codebook: int, workspace: torch.Tensor, normed: torch.Tensor | None = None) -> None:
    """residual += x (in place, when given); a = rmsnorm(residual or x) * weight; fragments of a for the following group;
    `normed` receives a when given.  All tensors share x's dtype (fp16 / bf16)."""
    _require_cuda(x, "x")
    rows, k = x.shape
    shards = suh_cat.numel() // k
    ws = _step_workspace(x.device, rows, k, shards, workspace)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().exl3_rmsnorm_rotate(_ptr(x), _ptr(residual), _ptr(weight), float(eps), _dtype_code(x), _ptr(suh_cat), shards,
                                                   rows, k, codebook, _ptr(normed), _ptr(ws), ws.numel(), _stream(x.device)),
                   "exl3_rmsnorm_rotate")


def silu_mul_rotate(gate_up: torch.Tensor, suh: torch.Tensor, codebook: int, workspace: torch.Tensor,
                    act: torch.Tensor | None = None) -> None:
    """a = silu(gate) * up of gate_up [rows, 2 * inter]; fragments of a for the following (down) matrix."""
    _require_cuda(gate_up, "gate_up")
    rows, two = gate_up.shape
    inter = two // 2
    ws = _step_workspace(gate_up.device, rows, inter, 1, workspace)
    with torch.cuda.device(gate_up.device):
        _lib.check(_lib.load().exl3_silu_mul_rotate(_ptr(gate_up), _dtype_code(gate_up), _ptr(suh), rows, inter, codebook, _ptr(act),
                                                    _ptr(ws), ws.numel(), _stream(gate_up.device)), "exl3_silu_mul_rotate")


def _residual_ptrs(residual):
    """residual = (stream in, stream out, sums of squares out) or None -> three pointers for the C ABI."""
    if residual is None:
        return None, None, None
    res_in, res_out, ssq_out = residual
    return _ptr(res_in), _ptr(res_out), _ptr(ssq_out)


def run_prerotated(rows: int, b: torch.Tensor, svh_cat: torch.Tensor, shard_ends: list[int], codebook: int, out: torch.Tensor | None,
                   workspace: torch.Tensor, exchange=None, residual=None, out_dtype: torch.dtype | None = None) -> torch.Tensor | None:
    """The fused group on the fragments the kernel ahead left in the workspace; `out` [rows, n_total] fp16 / bf16 (fp32:
    unrounded accumulators).  `exchange`: row-parallel shard, summed over the ranks inside the kernel.  `residual` =
    (stream in, stream out, sums of squares out float32 [rows, n_total / 128]): the epilogue carries the residual stream;
    `out` may then be None (give `out_dtype`)."""
    lib = _lib.load()
    _lib.init_device(b.device.index if b.device.index is not None else torch.cuda.current_device())
    k, n_total, K = _geometry(b)
    shards = len(shard_ends) + 1
    if workspace is None:
        raise RuntimeError("run_prerotated reads the fragments from the workspace the producing call wrote: pass that workspace")
    ws = _own_or_given(workspace, b.device, workspace_bytes(rows, k, n_total, shards), _workspace)
    ex = exchange if exchange is not None and exchange.world > 1 else None
    with torch.cuda.device(b.device):
        code = _dtype_code(out, True) if out is not None else _dtype_code(residual[1])
        _lib.check(lib.exl3_linear_prerotated(_ptr(b), K, codebook, _ptr(svh_cat), _lib.int_array(shard_ends), shards, rows, k, n_total,
                                              _ptr(out), code, _ptr(ws), ws.numel(),
                                              ex.peer_regions if ex else None, ex.rank if ex else 0, ex.world if ex else 1,
                                              ex.max_elems if ex else 0, _ptr(ex.state) if ex else None, *_residual_ptrs(residual),
                                              _stream(b.device)), "exl3_linear_prerotated")
    return out


def run_rmsnorm(x: torch.Tensor, residual_in: torch.Tensor | None, residual_out: torch.Tensor | None, weight: torch.Tensor, eps: float,
                b: torch.Tensor, suh_cat: torch.Tensor, svh_cat: torch.Tensor, shard_ends: list[int], codebook: int, out: torch.Tensor,
                workspace: torch.Tensor | None = None) -> torch.Tensor:
    """The fused group on rmsnorm(x + residual_in) * weight, with residual_out = x + residual_in written to a second buffer:
    `residual_ssq` followed by `run_normed`, for a caller whose stream does not come out of a linear's epilogue."""
    _require_cuda(x, "x")
    lib = _lib.load()
    _lib.init_device(b.device.index if b.device.index is not None else torch.cuda.current_device())
    k, n_total, K = _geometry(b)
    rows, shards = x.shape[0], len(shard_ends) + 1
    ws = _own_or_given(workspace, b.device, workspace_bytes(rows, k, n_total, shards), _workspace)
    with torch.cuda.device(b.device):
        _lib.check(lib.exl3_rmsnorm_linear(_ptr(x), _dtype_code(x), _ptr(residual_in), _ptr(residual_out), _ptr(weight), float(eps), _ptr(b), K,
                                           codebook, _ptr(suh_cat), _ptr(svh_cat), _lib.int_array(shard_ends), shards, rows, k, n_total,
                                           _ptr(out), _dtype_code(out, True), _ptr(ws), ws.numel(), _stream(b.device)), "exl3_rmsnorm_linear")
    return out


def residual_ssq(x: torch.Tensor, residual_in: torch.Tensor | None, residual_out: torch.Tensor | None, ssq: torch.Tensor) -> None:
    """z = x (+ residual_in) -> residual_out (optional) and the sums of squares of z per (row, 128 columns) -> ssq float32
    [rows, k / 128]: the start of a chain of residual blocks whose linears carry the stream in their epilogues."""
    _require_cuda(x, "x")
    rows, k = x.shape
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().exl3_residual_ssq(_ptr(x), _ptr(residual_in), _dtype_code(x), rows, k, _ptr(residual_out), _ptr(ssq),
                                                 _stream(x.device)), "exl3_residual_ssq")


def run_normed(z: torch.Tensor, ssq: torch.Tensor, weight: torch.Tensor, eps: float, b: torch.Tensor, suh_cat: torch.Tensor,
               svh_cat: torch.Tensor, shard_ends: list[int], codebook: int, out: torch.Tensor, workspace: torch.Tensor | None = None) -> torch.Tensor:
    """The fused group on rmsnorm(z) * weight, z a residual stream and ssq its sums of squares per 128 columns (from a linear's
    residual epilogue or `residual_ssq`): up to two rows the GEMV normalises on the way into its own rotation (one launch)."""
    _require_cuda(z, "z")
    lib = _lib.load()
    _lib.init_device(b.device.index if b.device.index is not None else torch.cuda.current_device())
    k, n_total, K = _geometry(b)
    rows, shards = z.shape[0], len(shard_ends) + 1
    ws = _own_or_given(workspace, b.device, workspace_bytes(rows, k, n_total, shards), _workspace)
    with torch.cuda.device(b.device):
        _lib.check(lib.exl3_normed_linear(_ptr(z), _dtype_code(z), _ptr(ssq), _ptr(weight), float(eps), _ptr(b), K, codebook, _ptr(suh_cat),
                                          _ptr(svh_cat), _lib.int_array(shard_ends), shards, rows, k, n_total, _ptr(out), _dtype_code(out, True),
                                          _ptr(ws), ws.numel(), _stream(b.device)), "exl3_normed_linear")
    return out


def run_glu(gate_up: torch.Tensor, b: torch.Tensor, suh: torch.Tensor, svh_cat: torch.Tensor, codebook: int, out: torch.Tensor | None,
            workspace: torch.Tensor | None = None, exchange=None, residual=None) -> torch.Tensor | None:
    """Down projection of silu(gate) * up straight from `gate_up` [rows, 2k]: up to two rows the activation is computed inside
    the GEMV's own input rotation (one launch, no activation buffer).  `exchange` and `residual` as in `run_prerotated`."""
    _require_cuda(gate_up, "gate_up")
    lib = _lib.load()
    _lib.init_device(b.device.index if b.device.index is not None else torch.cuda.current_device())
    k, n_total, K = _geometry(b)
    rows = gate_up.shape[0]
    if gate_up.shape[1] != 2 * k:
        raise ValueError(f"gate_up has {gate_up.shape[1]} columns, the matrix wants 2 x {k}")
    ws = _own_or_given(workspace, b.device, workspace_bytes(rows, k, n_total, 1), _workspace)
    ex = exchange if exchange is not None and exchange.world > 1 else None
    with torch.cuda.device(b.device):
        code = _dtype_code(out, True) if out is not None else _dtype_code(residual[1])
        _lib.check(lib.exl3_glu_linear(_ptr(gate_up), _dtype_code(gate_up), _ptr(b), K, codebook, _ptr(suh), _ptr(svh_cat), _lib.int_array([]), 1,
                                       rows, k, n_total, _ptr(out), code, _ptr(ws), ws.numel(),
                                       ex.peer_regions if ex else None, ex.rank if ex else 0, ex.world if ex else 1,
                                       ex.max_elems if ex else 0, _ptr(ex.state) if ex else None, *_residual_ptrs(residual),
                                       _stream(b.device)), "exl3_glu_linear")
    return out


# ---------------------------------------------------------------------------------------------------------------
# Building blocks (caller-owned buffers, rotated-basis product for reading decoded weights out, single matrices)

def reconstruct(trellis: torch.Tensor, codebook: int) -> torch.Tensor:
    """Stored trellis int16 (k/16, n/16, 16K) -> fp16 W_inner (k, n), bit-identical to the reference decoder."""
    _require_cuda(trellis, "trellis")
    lib = _lib.load()
    t = trellis.contiguous()
    kt, nt, words = t.shape
    w = torch.empty((kt * 16, nt * 16), dtype=torch.float16, device=t.device)
    with torch.cuda.device(t.device):
        _lib.check(lib.exl3_reconstruct(_ptr(t), kt * 16, nt * 16, words // 16, codebook, _ptr(w), _stream(t.device)),
                   "exl3_reconstruct")
    return w


def reconstruct_packed(packed: torch.Tensor, codebook: int) -> torch.Tensor:
    """Resident layout -> fp16 W_inner (k, n) through the same register-level decode the GEMV uses."""
    lib = _lib.load()
    k, n, K = _geometry(packed)
    w = torch.empty((k, n), dtype=torch.float16, device=packed.device)
    with torch.cuda.device(packed.device):
        _lib.check(lib.exl3_reconstruct_packed(_ptr(packed), k, n, K, codebook, _ptr(w), _stream(packed.device)),
                   "exl3_reconstruct_packed")
    return w


def had_in_group(x: torch.Tensor, suh_cat: torch.Tensor, xh: torch.Tensor | None = None) -> torch.Tensor:
    """xh[s] = Had128(fp16(x) * suh_cat[s]) for all shards in one launch: x [rows, k] -> fp16 [shards * rows, k]."""
    _require_cuda(x, "x")
    rows, k = x.shape
    shards = suh_cat.numel() // k
    if xh is None:
        xh = torch.empty((shards * rows, k), dtype=torch.float16, device=x.device)
    with torch.cuda.device(x.device):
        _lib.check(_lib.load().exl3_had_in(_ptr(x), _dtype_code(x), _ptr(suh_cat), shards, rows, k, _ptr(xh),
                                           _stream(x.device)), "exl3_had_in")
    return xh


def had_out_into(y: torch.Tensor, svh: torch.Tensor, out: torch.Tensor, col0: int) -> None:
    """out[:, col0:col0+n] = Had128(y) * svh in out's dtype (fp16 | bf16); y fp16 or fp32 [rows, n]."""
    _require_cuda(y, "y")
    rows, n = y.shape
    ydt = _lib.F32 if y.dtype == torch.float32 else _dtype_code(y)
    if col0 % 4 or out.stride(0) % 4:
        raise RuntimeError("col0 and the output row stride must be multiples of 4 elements")
    dst = ctypes.c_void_p(out.data_ptr() + col0 * out.element_size())
    with torch.cuda.device(y.device):
        _lib.check(_lib.load().exl3_had_out(_ptr(y), ydt, _ptr(svh), rows, n, dst, out.stride(0), _dtype_code(out),
                                            _stream(y.device)), "exl3_had_out")


def gemm_rotated_group(xh_all: torch.Tensor, packed: torch.Tensor, shard_ends, codebook: int,
                       out: torch.Tensor | None = None) -> torch.Tensor:
    """Rotated-basis product of a fused group; xh_all is (shards * rows, k) fp16, slab s feeds shard s.  An fp32 `out`
    receives the accumulators unrounded."""
    _require_cuda(xh_all, "xh")
    lib = _lib.load()
    _lib.init_device(xh_all.device.index if xh_all.device.index is not None else torch.cuda.current_device())
    k, n_total, K = _geometry(packed)
    shards = len(shard_ends) + 1
    rows = xh_all.shape[0] // shards
    if out is None:
        out = torch.empty((rows, n_total), dtype=torch.float16, device=xh_all.device)
    if rows == 0:
        return out
    ws = reserve_workspace(xh_all.device, workspace_bytes(rows, k, n_total, shards))
    fn = lib.exl3_gemm_rotated_f32 if out.dtype == torch.float32 else lib.exl3_gemm_rotated
    with torch.cuda.device(xh_all.device):
        _lib.check(fn(_ptr(xh_all), _ptr(packed), K, codebook, _lib.int_array(shard_ends), shards, rows,
                      k, n_total, _ptr(out), _ptr(ws), ws.numel(), _stream(xh_all.device)), "exl3_gemm_rotated")
    return out


def gemm_rotated(xh: torch.Tensor, packed: torch.Tensor, codebook: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """xh @ W_hat in the rotated basis (no Hadamards).  Identity rows of xh read W_hat out exactly."""
    return gemm_rotated_group(xh, packed, [], codebook, out)


def linear_group(x, packed, suh_cat, svh_cat, shard_ends, codebook: int, xh=None, out=None) -> torch.Tensor:
    """Fused group (output of `prepare`); `out` is (rows, sum(n)), shard s occupies its column span.  `xh` is accepted
    for signature compatibility and unused: the rotated input lives in the per-device workspace."""
    return run(x, packed, suh_cat, svh_cat, list(shard_ends), codebook, out)


def linear(x: torch.Tensor, packed: torch.Tensor, suh: torch.Tensor, svh: torch.Tensor, codebook: int,
           xh: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """One matrix: y = Had(x * suh) @ W_hat -> Had -> * svh."""
    return run(x, packed, suh.reshape(1, -1), svh, [], codebook, out)


def device_error(device: torch.device) -> None:
    """Raises if a bounded wait inside a kernel gave up since the last check (synchronises the stream)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspace.get(idx)
    if ws is not None:
        with torch.cuda.device(idx):
            _lib.check(_lib.load().exl3_device_error(_ptr(ws), ws.numel(), _stream(torch.device("cuda", idx))),
                       "exl3_device_error")


def set_tc_tiling(tiling: int) -> None:
    """Knob: output tiling of `run_tc`: -1 default, 0 tiles of 512 x 128, 1 of 256 x 256 (where the shape allows), 2 of 384 x 128,
    3 of 512 x 256 on pairs of CTAs (same condition as 1)."""
    _lib.load().exl3_set_tc_tiling(int(tiling))


def set_tc_ksplit(parts: int) -> None:
    """Knob: upper bound of the parts a tile's reduction is cut into in `run_tc` (0 default, 1 never split)."""
    _lib.load().exl3_set_tc_ksplit(int(parts))


def set_gemv_mode(mode: int) -> None:
    """Knob: -1 default, 0 split (two fp16 summands per weight, added in fp32), 1 paired (weights rounded to fp16)."""
    _lib.load().exl3_set_gemv_mode(int(mode))
