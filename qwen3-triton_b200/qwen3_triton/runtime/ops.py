"""FSDP2 pack / unpack data movement on the q3_multi_copy kernel.

FSDP2 moves every parameter of a unit three times per step through `torch.ops.fsdp.*`: the cast-and-pack of the
local fp32 shards into the bf16 all-gather input, the split of the all-gather output into per-parameter tensors,
and the chunk-and-upcast of the bf16 gradients into the fp32 reduce-scatter input. The stock CUDA implementations
run at 1-1.5 TB/s; `install_fsdp_pack_kernels()` replaces them (CUDA dispatch key only) with one q3_multi_copy
launch per call. Same role as the reference's runtime/ops.py:53-58,193-202 behind runtime/dispatch.py:105-119,
without a dispatch mode around the whole step.
"""
import math

import torch

from .. import _abi

_installed = False
_table_cache = {}
_seen_once = {}
_lib = None


def plan_copy_in(split_sizes, out_ptr, out_itemsize, rank, input_ptrs, input_numel=None):
    """Table rows for all_gather_copy_in: shard i -> its slice of this rank's all-gather input, which starts
    `input_numel` * rank elements into the output (input_numel = sum of the split sizes unless the caller says
    otherwise) and is cut by `split_sizes`."""
    first = (sum(split_sizes) if input_numel is None else input_numel) * rank
    rows, offset = [], 0
    for n, p in zip(split_sizes, input_ptrs):
        rows.append((p, out_ptr + (first + offset) * out_itemsize, 1, n, n, n, n))
        offset += n
    return rows


def plan_split(src_ptr, itemsize, world, split_sizes, out_ptrs):
    """Table rows for split_with_sizes_copy(dim=1) of a [world, total] buffer."""
    total = sum(split_sizes)
    rows, offset = [], 0
    for n, p in zip(split_sizes, out_ptrs):
        rows.append((src_ptr + offset * itemsize, p, world, n, total, n, (world - 1) * total + n))
        offset += n
    return rows


def plan_chunk_cat(shapes, src_ptrs, out_ptr, out_itemsize, world):
    """Table rows for chunk_cat(dim=0): tensor i is cut into `world` pieces of ceil(d0/world) leading rows
    (the tail zero-padded); piece r goes to out[r, offset_i : offset_i + piece_numel]. Returns (rows, out_cols)."""
    pieces = []
    for shape in shapes:
        d0 = shape[0] if len(shape) else 1
        rest = math.prod(shape[1:]) if len(shape) > 1 else 1
        pieces.append((-(-d0 // world)) * rest)
    out_cols = sum(pieces)
    rows, offset = [], 0
    for shape, piece, p in zip(shapes, pieces, src_ptrs):
        rows.append((p, out_ptr + offset * out_itemsize, world, piece, piece, out_cols, math.prod(shape) if len(shape) else 1))
        offset += piece
    return rows, out_cols


def finalize(rows):
    """Append vec_ok to each row; returns (table, total_elements). Empty pieces are dropped."""
    table, total = [], 0
    for src, dst, r, c, ss, ds, valid in rows:
        if r * c == 0:
            continue
        vec = int(c % 8 == 0 and ss % 8 == 0 and ds % 8 == 0 and src % 16 == 0 and dst % 16 == 0)
        table.append((src, dst, r, c, ss, ds, valid, vec))
        total += r * c
    return table, total


class _TableRing:
    """Device copies of tables whose pointers change from step to step (gradient buffers): a ring of pinned host
    slots and device slots, filled with an asynchronous copy on the launching stream, so that building a table
    never blocks the host on that stream. A slot is reused only after the launch that read it has finished."""
    SLOTS, ROWS = 64, 512

    def __init__(self, device):
        self.host = torch.empty((self.SLOTS, self.ROWS, 8), dtype=torch.int64, pin_memory=True)
        self.dev = torch.empty((self.SLOTS, self.ROWS, 8), dtype=torch.int64, device=device)
        self.events = [None] * self.SLOTS
        self.next = 0

    def put(self, table):
        slot = self.next
        self.next = (slot + 1) % self.SLOTS
        if self.events[slot] is not None:
            self.events[slot].synchronize()
        n = len(table)
        self.host[slot, :n] = torch.tensor(table, dtype=torch.int64)
        self.dev[slot, :n].copy_(self.host[slot, :n], non_blocking=True)
        return slot, self.dev[slot]

    def launched(self, slot):
        ev = self.events[slot] or torch.cuda.Event()
        ev.record()
        self.events[slot] = ev


_rings = {}


def _launch(rows, src_dtype, dst_dtype, device):
    table, total = finalize(rows)
    if not table:
        return
    key = tuple(table)
    meta = _table_cache.get(key)
    slot = None
    if meta is None and len(table) <= _TableRing.ROWS:
        seen = _seen_once.pop(key, None)
        if seen is None:
            # first sight: stream it through the ring; a table that comes back unchanged gets a permanent copy
            if len(_seen_once) > 4096:
                _seen_once.clear()
            _seen_once[key] = True
            ring = _rings.get(device)
            if ring is None:
                ring = _rings[device] = _TableRing(device)
            slot, meta = ring.put(table)
    if meta is None:
        if len(_table_cache) > 1024:
            _table_cache.clear()
        meta = torch.tensor(table, dtype=torch.int64).to(device)
        _table_cache[key] = meta
    _abi.call('q3_multi_copy', meta.data_ptr(), len(table), total, _abi.dt(src_dtype), _abi.dt(dst_dtype), _abi.stream())
    if slot is not None:
        _rings[device].launched(slot)


_FLOATS = (torch.float32, torch.bfloat16, torch.float16)


def all_gather_copy_in(all_gather_inputs, all_gather_output, inp_split_sizes, all_gather_input_numel, rank):
    all_gather_input = all_gather_output.narrow(0, all_gather_input_numel * rank, all_gather_input_numel)
    dtypes = {t.dtype for t in all_gather_inputs}
    sizes = [int(n) for n in inp_split_sizes]
    # the kernel path needs the split FSDP asked for to be the inputs' own sizes, filling this rank's slot exactly
    consistent = sizes == [t.numel() for t in all_gather_inputs] and sum(sizes) == all_gather_input_numel
    if (not consistent or len(dtypes) != 1 or next(iter(dtypes)) not in _FLOATS or all_gather_output.dtype not in _FLOATS
            or not all(t.is_contiguous() for t in all_gather_inputs)):
        with torch.no_grad():
            torch._foreach_copy_(torch.split(all_gather_input, inp_split_sizes), all_gather_inputs)
        return all_gather_input, all_gather_output
    rows = plan_copy_in(sizes, all_gather_output.data_ptr(), all_gather_output.element_size(), rank,
                        [t.data_ptr() for t in all_gather_inputs], all_gather_input_numel)
    _launch(rows, next(iter(dtypes)), all_gather_output.dtype, all_gather_output.device)
    return all_gather_input, all_gather_output


def launch_split_copy(all_gather_output, split_sizes, out):
    """The kernel form of split_with_sizes_copy(dim=1) on the current stream; False (nothing launched) for inputs it
    does not take."""
    ok = (all_gather_output.ndim == 2 and all_gather_output.is_contiguous() and len(out) > 0
          and all_gather_output.dtype in _FLOATS and len({o.dtype for o in out}) == 1 and out[0].dtype in _FLOATS
          and all(o.is_contiguous() and o.ndim == 2 for o in out))
    if not ok:
        return False
    rows = plan_split(all_gather_output.data_ptr(), all_gather_output.element_size(), all_gather_output.shape[0],
                      list(split_sizes), [o.data_ptr() for o in out])
    _launch(rows, all_gather_output.dtype, out[0].dtype, all_gather_output.device)
    return True


def split_with_sizes_copy(all_gather_output, all_gather_input_split_sizes, dim=0, *, out):
    if dim == 1 and all_gather_output.is_cuda:
        from .early_copy_out import pending_event
        event = pending_event(all_gather_output)
        if event is not None:           # copied ahead of time on the copy-out stream (runtime/early_copy_out.py)
            torch.cuda.current_stream(all_gather_output.device).wait_event(event)
            return
    if dim != 1 or not launch_split_copy(all_gather_output, all_gather_input_split_sizes, out):
        torch.split_with_sizes_copy(all_gather_output, all_gather_input_split_sizes, dim=dim, out=out)


_rs_root = None        # weak reference to the root FSDP module whose reduce-scatter stream takes the gradient pack
_peer_reducer = None   # runtime/peer_reduce.py:PeerGradientReducer when gradients are reduced over peer memory


def reduce_gradients_over_peer_memory(reducer):
    """With a PeerGradientReducer installed, `fsdp::chunk_cat` packs 16-bit gradients into its staging buffer (on the
    reduce-scatter stream) instead of upcasting them into FSDP's fp32 buffer; the reduce-scatter hook then pulls."""
    global _peer_reducer
    _peer_reducer = reducer


def pack_gradients_on_reduce_scatter_stream(root_module):
    """torch 2.11 issues the reduce-scatter copy-in (`fsdp::chunk_cat`) on the compute stream, where it costs about
    8 ms per step of Qwen3-8B. After this call the override runs it on FSDP's reduce-scatter stream instead, ordered
    after the compute stream's work so far; FSDP then queues the collective behind it on that same stream. The
    gradients are marked as used by that stream, so the allocator does not hand their memory out early."""
    global _rs_root
    import weakref
    _rs_root = weakref.ref(root_module) if root_module is not None else None


def _reduce_scatter_stream():
    root = _rs_root() if _rs_root is not None else None
    if root is None:
        return None
    try:
        ctx = root._get_fsdp_state()._comm_ctx
        return getattr(ctx, 'reduce_scatter_stream', None)
    except Exception:
        return None


def chunk_cat(tensors, dim, num_chunks, out):
    ok = (dim == 0 and out.ndim == 2 and out.is_contiguous() and out.dtype in _FLOATS and out.shape[0] == num_chunks
          and len({t.dtype for t in tensors}) == 1 and tensors[0].dtype in _FLOATS
          and all(t.is_contiguous() and t.ndim >= 1 for t in tensors))
    if ok:
        rows, cols = plan_chunk_cat([tuple(t.shape) for t in tensors], [t.data_ptr() for t in tensors], out.data_ptr(),
                                    out.element_size(), num_chunks)
        ok = cols == out.shape[1]
    if not ok:
        torch._chunk_cat(tensors, dim, num_chunks, out=out)
        return
    side = _reduce_scatter_stream()
    peer = _peer_reducer
    if peer is not None and (side is None or tensors[0].dtype not in (torch.bfloat16, torch.float16)
                             or out.dtype != torch.float32 or out.device != peer.device):
        peer = None
    if side is None:
        _launch(rows, tensors[0].dtype, out.dtype, out.device)
        return
    side.wait_stream(torch.cuda.current_stream(out.device))
    for t in tensors:
        t.record_stream(side)
    out.record_stream(side)
    with torch.cuda.stream(side):
        if peer is not None and peer.stage(tensors, out, _launch, plan_chunk_cat):
            return          # the gradients wait, still 16-bit, in the peer-visible staging buffer; `out` stays unwritten
        _launch(rows, tensors[0].dtype, out.dtype, out.device)


def install_fsdp_pack_kernels():
    """Route FSDP2's three pack/unpack ops to q3_multi_copy on CUDA tensors. Idempotent."""
    global _installed, _lib
    if _installed:
        return
    import torch.distributed.fsdp._fully_shard._fsdp_collectives  # noqa: F401  defines the fsdp:: ops
    _lib = torch.library.Library("fsdp", "IMPL")
    _lib.impl("all_gather_copy_in", all_gather_copy_in, "CUDA", allow_override=True)
    _lib.impl("split_with_sizes_copy", split_with_sizes_copy, "CUDA", allow_override=True)
    _lib.impl("chunk_cat", chunk_cat, "CUDA", allow_override=True)
    _installed = True
