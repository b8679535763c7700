"""Routed-expert (MoE) EXL3 layer on B200: the function surface of the reference's grouped backend
(cuda/src/sglang_exl3/kernels/marlin_moe.py of 0xSero/trellis-serve) over libexl3_b200's C ABI.

All experts of a projection are stacked `[E, ...]` in the resident layout of the dense kernel, gate and up
concatenated along n.  One layer is the reference's sequence (marlin_moe.py:272-294):

    had_in (gather, per-expert suh, 2 rotations) -> grouped GEMV gate|up (output transform inside the launch)
    -> glu_had_in (fp32 silu * up -> fp16 -> per-expert suh) -> grouped GEMV down -> fp32 router-weighted combine

Every (token, expert) slot has its own input rotation because every expert has its own suh (marlin_moe.py:11-13).
Routing is read on the device, so a captured CUDA graph replays with fresh routing.  Moe blocks are 8 rows of one
expert (`BLOCK_SIZES`); `align` here produces the (sorted_ids, expert_ids, num_post_padded) triple that the engine's
`moe_align_block_size` would, for that block size.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import torch

from .. import _lib
from .base import BackendStatus
from .linear import _dtype_code, _ptr, _require_cuda, _stream, prepare_matrix

BLOCK_SIZES = (8, 128)
# Average routed rows per expert from which a class goes through the grouped tensor-core GEMM (128-row blocks, every
# expert decoded once per up to 512 rows) instead of the grouped GEMV (8-row blocks, decoded once per block).
TC_ROWS_PER_EXPERT = 10
_workspace: dict[int, torch.Tensor] = {}


def probe() -> BackendStatus:
    try:
        lib = _lib.load()
    except (ImportError, OSError) as e:
        return BackendStatus(False, detail=str(e))
    return BackendStatus(True, version=str(lib.exl3_version()))


def moe_block_size(tokens: int, top_k: int, num_experts: int) -> int:
    """Rows per moe block.  The reference picks from a ladder 8..64 by T * top_k / E (marlin_moe.py:52-57); here decode-sized
    batches use the grouped GEMV on 8-row blocks and batches with many rows per expert the grouped tensor-core GEMM on
    128-row blocks (`run_layer` switches by this value)."""
    return BLOCK_SIZES[1] if tokens * top_k >= TC_ROWS_PER_EXPERT * num_experts else BLOCK_SIZES[0]


def sorted_ids_capacity(tokens: int, top_k: int, num_experts: int, block: int = 8) -> int:
    """Length of sorted_ids for these shapes (same bound as the engine's moe_align_block_size)."""
    return int(_lib.load().exl3_moe_sorted_capacity(tokens * top_k, num_experts))


def stack_repacked(trellis: list[torch.Tensor]) -> torch.Tensor:
    """E x int16 [k/16, n/16, 16K] -> int32 [E, n/128, k/128, 8, 2, K, 32]: a pure permutation of the stored words."""
    shapes = {tuple(t.shape) for t in trellis}
    if len(shapes) != 1:
        raise ValueError(f"experts must share one shape and bitrate, got {sorted(shapes)}")
    return torch.stack([prepare_matrix(t if t.is_cuda else t.cuda()) for t in trellis]).contiguous()


def bits_of_stack(stack: torch.Tensor) -> int:
    return stack.shape[-2]


@dataclass
class ExpertPack:
    w13: torch.Tensor      # int32 [E, 2I/128, H/128, 8, 2, K, 32]   gate | up along n
    w2: torch.Tensor       # int32 [E, H/128, I/128, 8, 2, K, 32]
    suh13: torch.Tensor    # fp16 [E, 2, H]
    svh13: torch.Tensor    # fp16 [E, 2I]
    suh2: torch.Tensor     # fp16 [E, I]
    svh2: torch.Tensor     # fp16 [E, H]
    codebook: int
    hidden: int
    inter: int
    num_experts: int
    bits: int = 4

    def tensors(self) -> list[torch.Tensor]:
        return [self.w13, self.w2, self.suh13, self.svh13, self.suh2, self.svh2]


def supports(gate: list[torch.Tensor], up: list[torch.Tensor], down: list[torch.Tensor], codebook: int) -> tuple[bool, str]:
    shapes = {tuple(t.shape) for t in gate} | {tuple(t.shape) for t in up}
    if len(shapes) != 1 or len({tuple(t.shape) for t in down}) != 1:
        return False, "experts differ in shape / bitrate"
    (kt, nt, words), (kt2, nt2, words2) = shapes.pop(), tuple(down[0].shape)
    if words != words2 or words % 16 or not 2 <= words // 16 <= 8:
        return False, "one integer K in 2..8 for all projections"
    if kt % 8 or nt % 8 or kt2 != nt or nt2 != kt:
        return False, "hidden / intermediate not multiples of 128, or down does not mirror gate/up"
    if codebook not in (0, 1, 2):
        return False, "codebook must be 3inst, mcg or mul1"
    return True, ""


def prepare(gate, up, down, codebook: int) -> ExpertPack:
    """gate / up / down = (trellis list, suh list, svh list) indexed by expert.  Pure re-layout, no value changes."""
    dev = gate[0][0].device
    if dev.type != "cuda":
        dev = torch.device("cuda", torch.cuda.current_device())
    _lib.init_device(dev.index)
    w13 = torch.cat([stack_repacked(gate[0]), stack_repacked(up[0])], dim=1).contiguous()
    w2 = stack_repacked(down[0])
    suh13 = torch.stack([torch.stack(gate[1]), torch.stack(up[1])], dim=1).contiguous().to(dev)
    svh13 = torch.cat([torch.stack(gate[2]), torch.stack(up[2])], dim=1).contiguous().to(dev)
    suh2, svh2 = torch.stack(down[1]).contiguous().to(dev), torch.stack(down[2]).contiguous().to(dev)
    hidden, inter = w13.shape[2] * 128, w2.shape[2] * 128
    return ExpertPack(w13, w2, suh13, svh13, suh2, svh2, codebook, hidden, inter, w13.shape[0], bits_of_stack(w13))


@dataclass
class MixedPack:
    """Experts of mixed K (e.g. 192 experts at K = 3 and 64 at K = 4 in one layer), the reference's `MixedPack`
    (marlin_moe.py:135-161): one ExpertPack per bitrate class in LOCAL expert order and, per class, the map global id ->
    local id (-1 elsewhere).  Every slot belongs to exactly one class, so the classes' grouped GEMVs together fill the
    shared gate|up and down slabs; one router-weighted combine closes the layer."""
    packs: list[ExpertPack]
    expert_maps: list[torch.Tensor]     # int32 [E] per class: global id -> local id, -1 elsewhere
    num_experts: int
    hidden: int
    inter: int
    codebook: int
    expert_ids: list[torch.Tensor] = field(default_factory=list)    # int32 [E_c] per class: local id -> global id
    covers_all: bool = True             # False: some experts belong to no class (another rank holds them)

    def __post_init__(self):
        if not self.expert_ids:
            self.expert_ids = [(m >= 0).nonzero().flatten().to(torch.int32).contiguous() for m in self.expert_maps]

    @property
    def bits(self) -> list[int]:
        return [p.bits for p in self.packs]

    def block_sizes(self, tokens: int, top_k: int) -> list[int]:
        return [moe_block_size(tokens, top_k, p.num_experts) for p in self.packs]


def prepare_mixed(gate, up, down, codebook: int, experts=None) -> MixedPack:
    """Like `prepare`, for experts of mixed K (marlin_moe.py:164-181): experts are grouped by their bitrate.  `experts`
    (an iterable of global expert ids) restricts the pack to those experts: the slots of all others belong to no class,
    which is how one rank of an expert-parallel layer holds its share (`expert_partition`)."""
    words = [w.shape[2] for w in gate[0]]
    e = len(words)
    keep = sorted(set(range(e) if experts is None else experts))
    if not keep or keep[0] < 0 or keep[-1] >= e:
        raise ValueError(f"experts must be a non-empty subset of 0..{e - 1}")
    classes = sorted({words[i] for i in keep})
    packs, maps = [], []
    for wd in classes:
        ids = [i for i in keep if words[i] == wd]
        sub = lambda t: tuple([t[j][i] for i in ids] for j in range(3))
        packs.append(prepare(sub(gate), sub(up), sub(down), codebook))
        m = torch.full((e,), -1, dtype=torch.int32)
        m[ids] = torch.arange(len(ids), dtype=torch.int32)
        maps.append(m.to(packs[-1].w13.device))
    return MixedPack(packs, maps, e, packs[0].hidden, packs[0].inter, codebook, covers_all=len(keep) == e)


def expert_partition(num_experts: int, rank: int, world: int) -> range:
    """Experts of one rank under expert parallelism: contiguous shares, the first `num_experts % world` ranks take one
    more.  Tokens are replicated, every rank computes the weighted contributions of its own experts and the outputs
    [T, hidden] are summed by one all-reduce."""
    if not 0 <= rank < world or num_experts < world:
        raise ValueError(f"cannot split {num_experts} experts over rank {rank} of {world}")
    q, r = divmod(num_experts, world)
    lo = rank * q + min(rank, r)
    return range(lo, lo + q + (1 if rank < r else 0))


def align_capacity(slots: int, num_experts_class: int, block: int = 8) -> int:
    """Length of sorted_ids for one class (marlin_moe.py:186-192 gives the engine's bound; this is the library's)."""
    return int(_lib.load().exl3_moe_sorted_capacity(slots, num_experts_class))


def align_decode(topk_ids: torch.Tensor, pack: MixedPack, tokens: int, top_k: int) -> list[tuple]:
    """Routings for run_mixed (marlin_moe.py:195-213): per class (sorted_ids, expert_ids, num_post, block) over that
    class's slots only, expert ids local to the class."""
    _require_cuda(topk_ids, "topk_ids")
    lib = _lib.load()
    ids = topk_ids.reshape(-1).to(torch.int32).contiguous()
    out = []
    with torch.cuda.device(ids.device):
        for pk, emap in zip(pack.packs, pack.expert_maps):
            cap = align_capacity(ids.numel(), pk.num_experts)
            sorted_ids = torch.empty((cap,), dtype=torch.int32, device=ids.device)
            expert_ids = torch.empty((max(cap // 8, 1),), dtype=torch.int32, device=ids.device)
            num_post = torch.empty((1,), dtype=torch.int32, device=ids.device)
            _lib.check(lib.exl3_moe_align_mapped(_ptr(ids), ids.numel(), pack.num_experts, _ptr(emap), pk.num_experts, _ptr(sorted_ids),
                                                 cap, _ptr(expert_ids), _ptr(num_post), _stream(ids.device)), "exl3_moe_align_mapped")
            out.append((sorted_ids, expert_ids, num_post, 8))
    return out


def _reserve(device: torch.device, nbytes: int) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    cur = _workspace.get(idx)
    if cur is None or cur.numel() < nbytes:
        cur = _workspace[idx] = torch.zeros(nbytes, dtype=torch.uint8, device=torch.device("cuda", idx))
    return cur


def align(topk_ids: torch.Tensor, num_experts: int, block: int = 8):
    """-> (sorted_ids int32 [cap], expert_ids int32 [cap / 8], num_post_padded int32 [1]), computed on the device."""
    _require_cuda(topk_ids, "topk_ids")
    lib = _lib.load()
    ids = topk_ids.reshape(-1).to(torch.int32).contiguous()
    cap = int(lib.exl3_moe_sorted_capacity(ids.numel(), num_experts))
    sorted_ids = torch.empty((cap,), dtype=torch.int32, device=ids.device)
    expert_ids = torch.empty((max(cap // 8, 1),), dtype=torch.int32, device=ids.device)
    num_post = torch.empty((1,), dtype=torch.int32, device=ids.device)
    with torch.cuda.device(ids.device):
        _lib.check(lib.exl3_moe_align(_ptr(ids), ids.numel(), num_experts, _ptr(sorted_ids), cap, _ptr(expert_ids), _ptr(num_post),
                                      _stream(ids.device)), "exl3_moe_align")
    return sorted_ids, expert_ids, num_post


def gemm_rotated(xf, stack, out, sorted_ids, expert_ids, num_post_padded, slots: int, shard_end: int, codebook: int,
                 svh=None) -> torch.Tensor:
    """Grouped product (svh=None: rotated basis, no output transform).  xf = activation fragments of the blocks."""
    lib = _lib.load()
    e, nb, kg, _, _, K, _ = stack.shape
    k, n_total, cap = kg * 128, nb * 128, sorted_ids.numel()
    ws = _reserve(stack.device, int(lib.exl3_moe_workspace_bytes(cap, n_total)))
    with torch.cuda.device(stack.device):
        _lib.check(lib.exl3_moe_gemm(_ptr(xf), _ptr(stack), K, codebook, _ptr(svh), _ptr(sorted_ids), _ptr(expert_ids),
                                     _ptr(num_post_padded), cap, slots, k, n_total, shard_end, _ptr(out), _ptr(ws), ws.numel(),
                                     _stream(stack.device)), "exl3_moe_gemm")
    return out


def run_tensors(x, topk_weights, topk_ids, sorted_ids, expert_ids, num_post_padded, block: int, w13, w2, suh13, svh13,
                suh2, svh2, codebook: int, out: torch.Tensor | None = None) -> torch.Tensor:
    """x fp16 | bf16 [T, H]; topk_weights float32 [T, top_k]; topk_ids int32 | int64 [T, top_k]; routing triple from
    `align` (or the engine's moe_align_block_size with block 8).  -> y [T, H] in x's dtype."""
    _require_cuda(x, "x")
    lib = _lib.load()
    tokens, hidden = x.shape
    top_k, inter = topk_ids.shape[1], suh2.shape[1]
    slots = tokens * top_k
    y = out if out is not None else torch.empty_like(x)
    if tokens == 0:
        return y
    if block != 8:
        raise RuntimeError(f"the grouped GEMV works on 8-row moe blocks, got block = {block}")
    dev, st = x.device, _stream(x.device)
    cap = sorted_ids.numel()
    ids32 = topk_ids.reshape(-1).to(torch.int32).contiguous()
    wts = topk_weights.reshape(-1).to(torch.float32).contiguous()
    xf13 = torch.empty(int(lib.exl3_moe_fragment_bytes(cap, hidden, 2, codebook)), dtype=torch.uint8, device=dev)
    gu = torch.empty((slots, 2 * inter), dtype=torch.float16, device=dev)
    xf2 = torch.empty(int(lib.exl3_moe_fragment_bytes(cap, inter, 1, codebook)), dtype=torch.uint8, device=dev)
    yd = torch.empty((slots, hidden), dtype=torch.float16, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.exl3_moe_had_in(_ptr(x), _dtype_code(x), _ptr(suh13), 2, hidden, top_k, slots, _ptr(sorted_ids), cap,
                                       _ptr(expert_ids), _ptr(num_post_padded), codebook, _ptr(xf13), st), "exl3_moe_had_in")
    gemm_rotated(xf13, w13, gu, sorted_ids, expert_ids, num_post_padded, slots, inter, codebook, svh13)
    with torch.cuda.device(dev):
        _lib.check(lib.exl3_moe_glu_had_in(_ptr(gu), _ptr(suh2), inter, slots, _ptr(sorted_ids), cap, _ptr(expert_ids),
                                           _ptr(num_post_padded), codebook, _ptr(xf2), st), "exl3_moe_glu_had_in")
    gemm_rotated(xf2, w2, yd, sorted_ids, expert_ids, num_post_padded, slots, 0, codebook, svh2)
    with torch.cuda.device(dev):
        _lib.check(lib.exl3_moe_combine(_ptr(yd), _ptr(wts), _ptr(ids32), tokens, top_k, hidden, w13.shape[0], _ptr(y),
                                        _dtype_code(y), st), "exl3_moe_combine")
    return y


def run_mixed(x, topk_weights, topk_ids, routings, pack: MixedPack, out: torch.Tensor | None = None) -> torch.Tensor:
    """One MoE layer over experts of mixed K (marlin_moe.py:247-269).  routings = `align_decode(...)`.  Per class the
    input rotation uses the class's own sign vectors and routing, the grouped GEMVs write that class's slots of the
    shared gate|up and down slabs, and one combine over all slots closes the layer."""
    _require_cuda(x, "x")
    lib = _lib.load()
    tokens, hidden = x.shape
    top_k, inter = topk_ids.shape[1], pack.inter
    slots = tokens * top_k
    y = out if out is not None else torch.empty_like(x)
    if tokens == 0:
        return y
    dev, st = x.device, _stream(x.device)
    ids32 = topk_ids.reshape(-1).to(torch.int32).contiguous()
    wts = topk_weights.reshape(-1).to(torch.float32).contiguous()
    gu = torch.empty((slots, 2 * inter), dtype=torch.float16, device=dev)
    # slots of experts that no class of this pack holds are never written: they must add nothing in the combine
    yd = (torch.empty if pack.covers_all else torch.zeros)((slots, hidden), dtype=torch.float16, device=dev)
    for pk, (sorted_ids, expert_ids, num_post, block) in zip(pack.packs, routings):
        if block != 8:
            raise RuntimeError(f"the grouped GEMV works on 8-row moe blocks, got block = {block}")
        cap = sorted_ids.numel()
        xf13 = torch.empty(int(lib.exl3_moe_fragment_bytes(cap, hidden, 2, pk.codebook)), dtype=torch.uint8, device=dev)
        xf2 = torch.empty(int(lib.exl3_moe_fragment_bytes(cap, inter, 1, pk.codebook)), dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            _lib.check(lib.exl3_moe_had_in(_ptr(x), _dtype_code(x), _ptr(pk.suh13), 2, hidden, top_k, slots, _ptr(sorted_ids), cap,
                                           _ptr(expert_ids), _ptr(num_post), pk.codebook, _ptr(xf13), st), "exl3_moe_had_in")
        gemm_rotated(xf13, pk.w13, gu, sorted_ids, expert_ids, num_post, slots, inter, pk.codebook, pk.svh13)
        with torch.cuda.device(dev):
            _lib.check(lib.exl3_moe_glu_had_in(_ptr(gu), _ptr(pk.suh2), inter, slots, _ptr(sorted_ids), cap, _ptr(expert_ids),
                                               _ptr(num_post), pk.codebook, _ptr(xf2), st), "exl3_moe_glu_had_in")
        gemm_rotated(xf2, pk.w2, yd, sorted_ids, expert_ids, num_post, slots, 0, pk.codebook, pk.svh2)
    with torch.cuda.device(dev):
        _lib.check(lib.exl3_moe_combine(_ptr(yd), _ptr(wts), _ptr(ids32), tokens, top_k, hidden, pack.num_experts, _ptr(y),
                                        _dtype_code(y), st), "exl3_moe_combine")
    return y


def forward_mixed(x, topk_weights, topk_ids, pack: MixedPack, out: torch.Tensor | None = None) -> torch.Tensor:
    """Whole mixed-K layer including the per-class routing alignment."""
    return run_mixed(x, topk_weights, topk_ids, align_decode(topk_ids, pack, x.shape[0], topk_ids.shape[1]), pack, out)


def forward_expert_parallel(x, topk_weights, topk_ids, pack: MixedPack, reduce, out: torch.Tensor | None = None) -> torch.Tensor:
    """One rank of an expert-parallel layer: `pack` holds this rank's experts (`prepare_mixed(..., experts=
    expert_partition(E, rank, world))`), tokens and routing are the same on every rank, `reduce` sums a tensor over the
    ranks in place (`runtime.allreduce.PeerAllReduce` or `nccl_all_reduce`)."""
    y = forward_mixed(x, topk_weights, topk_ids, pack, out)
    reduce(y)
    return y


# ---------------------------------------------------------------------------------------------------------------
# One layer with every temporary carved out of a caller-owned workspace: the form the backend contract asks for
# (cuda/src/sglang_exl3/kernels/base.py:74-80: after warm-up the run path never allocates).

def _up256(n: int) -> int:
    return (n + 255) & ~255


def _layer_regions(num_experts_per_class: list[int], hidden: int, inter: int, codebook: int, tokens: int, top_k: int):
    """[(name, nbytes)] of one layer's temporaries, in workspace order; per class: routing triple and fragment buffers."""
    lib = _lib.load()
    slots = tokens * top_k
    regions = [("ids32", slots * 4), ("wts", slots * 4), ("gu", slots * 2 * inter * 2), ("yd", slots * hidden * 2)]
    gemv = 0
    for c, e in enumerate(num_experts_per_class):
        cap = int(lib.exl3_moe_sorted_capacity(slots, e))
        regions += [(f"sorted{c}", cap * 4), (f"experts{c}", max(cap // 8, 1) * 4), (f"post{c}", 4),
                    (f"xf13_{c}", int(lib.exl3_moe_fragment_bytes(cap, hidden, 2, codebook))),
                    (f"xf2_{c}", int(lib.exl3_moe_fragment_bytes(cap, inter, 1, codebook)))]
        gemv = max(gemv, int(lib.exl3_moe_workspace_bytes(cap, 2 * inter)), int(lib.exl3_moe_workspace_bytes(cap, hidden)))
        if moe_block_size(tokens, top_k, e) == BLOCK_SIZES[1]:
            regions.append((f"tc{c}", int(lib.exl3_moe_tc_workspace_bytes(slots, e, hidden, inter))))
    return [("gemv", gemv)] + regions       # the GEMV workspace first: its header and counters must stay zero


def layer_workspace_bytes(num_experts_per_class: list[int], hidden: int, inter: int, codebook: int, tokens: int, top_k: int) -> int:
    """Bytes `run_layer` needs for up to `tokens` tokens (zero-filled once by the caller)."""
    return sum(_up256(n) for _, n in _layer_regions(num_experts_per_class, hidden, inter, codebook, tokens, top_k))


def run_layer(x, topk_weights, topk_ids, pack: MixedPack, out: torch.Tensor, workspace: torch.Tensor,
              expert_maps: list[torch.Tensor] | None = None) -> torch.Tensor:
    """One MoE layer (alignment included) that allocates nothing: `workspace` is a zero-filled uint8 tensor of at least
    `layer_workspace_bytes(...)`; `expert_maps` replaces the pack's per-class maps (expert parallelism with an engine's
    global -> local map composed in).  Same kernels and the same bits as `forward_mixed` for decode-sized batches; a class
    whose experts see `TC_ROWS_PER_EXPERT` rows or more on average goes through the grouped tensor-core GEMM."""
    _require_cuda(x, "x")
    lib = _lib.load()
    tokens, hidden = x.shape
    top_k, inter = topk_ids.shape[1], pack.inter
    slots = tokens * top_k
    if tokens == 0:
        return out
    dev, st = x.device, _stream(x.device)
    maps = expert_maps if expert_maps is not None else pack.expert_maps
    views, off = {}, 0
    for name, n in _layer_regions([p.num_experts for p in pack.packs], hidden, inter, pack.codebook, tokens, top_k):
        views[name] = workspace[off:off + n]
        off += _up256(n)
    if off > workspace.numel():
        raise RuntimeError(f"MoE workspace holds {workspace.numel()} bytes, this call needs {off}")
    ids32, wts = views["ids32"].view(torch.int32), views["wts"].view(torch.float32)
    ids32.copy_(topk_ids.reshape(-1))
    wts.copy_(topk_weights.reshape(-1))
    gu, yd, ws = views["gu"], views["yd"], views["gemv"]
    if not pack.covers_all or expert_maps is not None:
        yd.zero_()                        # slots of experts held elsewhere are never written and must add nothing
    with torch.cuda.device(dev):
        for c, (pk, emap) in enumerate(zip(pack.packs, maps)):
            sorted_ids, expert_ids, num_post = views[f"sorted{c}"], views[f"experts{c}"], views[f"post{c}"]
            xf13, xf2 = views[f"xf13_{c}"], views[f"xf2_{c}"]
            cap = sorted_ids.numel() // 4
            K = pk.bits
            if moe_block_size(tokens, top_k, pk.num_experts) == BLOCK_SIZES[1]:
                tc = views[f"tc{c}"]
                tc[:256].zero_()          # this region moves with the token count: its error word starts clean
                _lib.check(lib.exl3_moe_tc_experts(_ptr(x), _dtype_code(x), tokens, top_k, hidden, inter, _ptr(ids32), emap.numel(), _ptr(emap),
                                                   pk.num_experts, _ptr(pk.w13), _ptr(pk.suh13), _ptr(pk.svh13), _ptr(pk.w2), _ptr(pk.suh2),
                                                   _ptr(pk.svh2), K, pk.codebook, _ptr(yd), _ptr(tc), tc.numel(), st), "exl3_moe_tc_experts")
                continue
            _lib.check(lib.exl3_moe_align_mapped(_ptr(ids32), slots, emap.numel(), _ptr(emap), pk.num_experts, _ptr(sorted_ids), cap,
                                                 _ptr(expert_ids), _ptr(num_post), st), "exl3_moe_align_mapped")
            _lib.check(lib.exl3_moe_had_in(_ptr(x), _dtype_code(x), _ptr(pk.suh13), 2, hidden, top_k, slots, _ptr(sorted_ids), cap,
                                           _ptr(expert_ids), _ptr(num_post), pk.codebook, _ptr(xf13), st), "exl3_moe_had_in")
            _lib.check(lib.exl3_moe_gemm(_ptr(xf13), _ptr(pk.w13), K, pk.codebook, _ptr(pk.svh13), _ptr(sorted_ids), _ptr(expert_ids),
                                         _ptr(num_post), cap, slots, hidden, 2 * inter, inter, _ptr(gu), _ptr(ws), ws.numel(), st),
                       "exl3_moe_gemm")
            _lib.check(lib.exl3_moe_glu_had_in(_ptr(gu), _ptr(pk.suh2), inter, slots, _ptr(sorted_ids), cap, _ptr(expert_ids),
                                               _ptr(num_post), pk.codebook, _ptr(xf2), st), "exl3_moe_glu_had_in")
            _lib.check(lib.exl3_moe_gemm(_ptr(xf2), _ptr(pk.w2), K, pk.codebook, _ptr(pk.svh2), _ptr(sorted_ids), _ptr(expert_ids),
                                         _ptr(num_post), cap, slots, inter, hidden, 0, _ptr(yd), _ptr(ws), ws.numel(), st),
                       "exl3_moe_gemm")
        _lib.check(lib.exl3_moe_combine(_ptr(yd), _ptr(wts), _ptr(ids32), tokens, top_k, hidden, maps[0].numel(), _ptr(out),
                                        _dtype_code(out), st), "exl3_moe_combine")
    return out


def run(x, topk_weights, topk_ids, sorted_ids, expert_ids, num_post_padded, block: int, pack: ExpertPack,
        out: torch.Tensor | None = None) -> torch.Tensor:
    return run_tensors(x, topk_weights, topk_ids, sorted_ids, expert_ids, num_post_padded, block, *pack.tensors(),
                       pack.codebook, out)


def forward(x, topk_weights, topk_ids, pack: ExpertPack, out: torch.Tensor | None = None) -> torch.Tensor:
    """Whole layer including the routing alignment."""
    s, e, p = align(topk_ids, pack.num_experts)
    return run(x, topk_weights, topk_ids, s, e, p, 8, pack, out)
