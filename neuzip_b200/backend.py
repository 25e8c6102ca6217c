"""Python stand-in for the reference's native module ``neuzip._cuda``
(cuda/neuzip.cu:19-106): an ``Algorithm`` enum and the backend classes
``Manager_f{precision}_n{normalizer}`` with ``read / write / size / linear /
linear_without_bias / split`` (cuda/neuzip.cu:28-37).

Where the reference keeps its compressed tensors in a C++ map inside the
extension (cuda/high_level.cu:35-43), this backend keeps torch tensors in a
Python dict and calls the stateless C-ABI kernels of ``libneuzip_b200.so`` on
the caller's current CUDA stream.  Only the rANS ("ans") algorithm, bf16
tensors are implemented (every precision and normaliser size); the other
algorithms raise ``NotImplementedError`` when constructed.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import ctypes

import torch

from . import _lib

PRECISIONS = (0, 1, 3, 7)
NORMALIZER_SIZES = (0, 1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024)


class Algorithm(enum.Enum):
    """Same members, same order as the extension enum (cuda/algorithms.cuh:8)."""
    ans = 0
    bitcomp = 1
    lz4 = 2
    zstd = 3
    gdeflate = 4


@dataclass
class _Entry:
    numel: int
    dtype: torch.dtype
    lane_symbols: int
    max_unit_words: int
    container: torch.Tensor   # uint8, right-sized NZR1 container
    fractions: torch.Tensor   # uint8, packed sign+mantissa stream
    normalizers: Optional[torch.Tensor] = None   # uint8, one byte per group (normalizer_size > 0)
    stamp: int = 0            # number of the library operation that wrote these bytes
    operand_cols: int = 0     # > 0: a [numel / operand_cols, operand_cols] matrix in operand order
    # While a write is still in flight the container sits in its worst-case-sized buffer;
    # `pending` = (slot of the pinned header copy, event after that copy).  Once the event has
    # completed the entry is settled: right-sized container, real max_unit_words.
    pending: Optional[tuple] = None
    version: int = 0          # bumped when the container tensor is replaced


# Every operation that any backend of this process enqueues gets a number.  A decode
# may promise NZ_ITEM_INPUTS_STABLE for an entry only when some other operation was
# enqueued between the entry's write and the decode: then the write is not "the work
# enqueued just before the call", whichever Manager or handle it went through.
_op_counter = 0


def _next_op() -> int:
    global _op_counter
    _op_counter += 1
    return _op_counter


def _stable_flag(entries, op: int) -> int:
    return _lib.NZ_ITEM_INPUTS_STABLE if all(e.stamp < op - 1 for e in entries) else 0


class _Batch:
    """Argument blocks of a batched decode, rebuilt when an entry is replaced."""
    __slots__ = ("names", "outs", "entries", "versions", "blocks", "lane_symbols")

    def __init__(self, names, outs) -> None:
        self.names = list(names)
        self.outs = list(outs)
        self.entries = []
        self.versions = []
        self.blocks = None
        self.lane_symbols = 0


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_bf16(tensor: torch.Tensor) -> None:
    if tensor.dtype != torch.bfloat16:
        # the reference dispatches fp32/fp16 as well (cuda/high_level.cu:144-158) but
        # truncates their mantissa to 8 bits (cuda/kernels.cuh:123); only bf16 is sound
        raise RuntimeError("Unsupported data type")


def _as_flat_bf16_cuda(tensor: torch.Tensor) -> torch.Tensor:
    _require_bf16(tensor)
    if not tensor.is_cuda:
        tensor = tensor.cuda()
    flat = tensor.detach().contiguous().view(-1)
    if flat.data_ptr() % 16:
        flat = flat.clone()
    return flat


class CodecBackend:
    """One (precision, normalizer) instantiation of the reference's C++
    ``Manager`` template (cuda/high_level.cu:26-322)."""

    precision: int = 7
    normalizer_size: int = 0
    supports_operand_order = True      # write() takes operand=

    def __init__(self, algorithm: Algorithm = Algorithm.ans, chunk_size: int = 1 << 16) -> None:
        if not isinstance(algorithm, Algorithm):
            algorithm = Algorithm(algorithm)
        if algorithm is not Algorithm.ans:
            raise NotImplementedError(
                f"algorithm {algorithm.name!r}: only the rANS coder ('ans') is implemented")
        self._lib = _lib.load()
        self.chunk_size = int(chunk_size)   # kept for API parity; the unit size follows precision
        self.lane_symbols = int(self._lib.nz_default_lane_symbols(self.precision))
        self._cache: Dict[str, _Entry] = {}
        self._scratch: Optional[torch.Tensor] = None
        self._status: Optional[torch.Tensor] = None
        self.canonical_nan = True           # NaN -> 0x7FFF like cuda/kernels.cuh:214-216
        # single-vector linear calls multiply while decoding (see _linear_vec); off by
        # default because the sums are ordered differently from the library GEMM's
        self.fused_vector_linear = False
        self._vec_src: Optional[torch.Tensor] = None
        self._vec_ver = -1
        self._vec_x: Optional[torch.Tensor] = None
        self._vec_scratch: Dict[tuple, torch.Tensor] = {}
        # 2-D weights written with operand=True are stored in operand order when their shape
        # allows it (the stream's 256-element blocks are 4 x 64 patches of the matrix), which
        # is what lets `linear` decode straight into tensor-core operand tiles
        self.operand_order = True
        # `linear` with at most this many input rows runs the fused decode -> tcgen05 GEMM
        # (nz_linear_bf16) on operand-order weights; 0 = always decode, then library GEMM
        self.fused_linear_max_rows = 0
        self._lin_ws: Optional[torch.Tensor] = None
        # pinned header slots and events of writes that have not been right-sized yet
        self._hdr_chunks: List[torch.Tensor] = []
        self._hdr_base: List[int] = []
        self._hdr_free: List[int] = []
        self._event_pool: list = []
        # True: `write` waits for the compressed size like the reference does
        self.sync_writes = False

    # -- helpers ---------------------------------------------------------
    def _ensure_device(self) -> None:
        if self._status is None:
            _lib.check(self._lib.nz_device_check())
            self._status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def _scratch_for(self, nbytes: int) -> torch.Tensor:
        if self._scratch is None or self._scratch.numel() < nbytes:
            self._scratch = None
            self._scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        return self._scratch

    def release_scratch(self) -> None:
        self._scratch = None

    def status(self) -> int:
        """Decode status word accumulated so far (synchronises)."""
        return 0 if self._status is None else int(self._status.item()) & 0xFFFFFFFF

    def check(self) -> None:
        word = self.status()
        if word:
            raise _lib.NeuzipError("decode reported: " + _lib.describe_status(word))

    # -- the six methods of the extension class ----------------------------
    def _operand_geometry(self, tensor: torch.Tensor):
        """(cols, lane_symbols) for a matrix that can be stored in operand order, else None."""
        if tensor.dim() != 2 or self.normalizer_size:
            return None          # group scales follow the flat element index
        rows, cols = int(tensor.shape[0]), int(tensor.shape[1])
        if rows % 4 or cols % 64:
            return None
        S = int(self._lib.nz_operand_lane_symbols_for(rows, cols, self.precision))
        return (cols, S) if S else None

    def write(self, name: str, tensor: torch.Tensor, operand: Optional[bool] = None) -> None:
        """cuda/high_level.cu:132-162 (+ _write_to_cache :71-130).  `operand=True` asks for
        operand order (a Linear weight); None keeps the layout the handle already has."""
        _require_bf16(tensor)
        self._ensure_device()
        flat = _as_flat_bf16_cuda(tensor)
        n = flat.numel()
        L, S = self._lib, self.lane_symbols
        previous = self._cache.pop(name, None)
        if operand is None:
            operand = previous is not None and previous.operand_cols > 0
        geometry = self._operand_geometry(tensor) if (operand and self.operand_order) else None
        if (geometry is None and operand and previous is not None and previous.operand_cols
                and tensor.dim() != 2 and n % previous.operand_cols == 0):
            # an update of an operand-order weight that arrives flattened
            geometry = self._operand_geometry(tensor.reshape(-1, previous.operand_cols))
        st = _stream()
        if geometry is not None:
            cols, S = geometry
            rows = n // cols
            frac = torch.empty(int(L.nz_frac_bytes(n, self.precision)), dtype=torch.uint8, device="cuda")
            cap = int(L.nz_container_bound(n, S))
            staging = torch.empty(cap, dtype=torch.uint8, device="cuda")
            scratch = self._scratch_for(int(L.nz_compress_operand_scratch_bytes(rows, cols, S)))
            _lib.check(L.nz_compress_bf16_operand(_ptr(flat), rows, cols, self.precision, S,
                                                  _ptr(frac), _ptr(staging), cap, _ptr(scratch),
                                                  scratch.numel(), st))
            self._cache[name] = self._finish_write(
                _Entry(n, tensor.dtype, S, 0, staging, frac, None, _next_op(), cols), previous)
            return
        normalizers = None
        if self.normalizer_size:
            # per-group scaling first (cuda/kernels.cuh:94-118); the scaled copy is what gets split
            normalizers = torch.empty(int(L.nz_normalizer_bytes(n, self.normalizer_size)),
                                      dtype=torch.uint8, device="cuda")
            scaled = torch.empty_like(flat)
            _lib.check(L.nz_normalize_bf16(_ptr(flat), n, self.normalizer_size, _ptr(scaled),
                                           _ptr(normalizers), st))
            flat = scaled
        frac = torch.empty(int(L.nz_frac_bytes(n, self.precision)), dtype=torch.uint8, device="cuda")
        cap = int(L.nz_container_bound(n, S))
        staging = torch.empty(cap, dtype=torch.uint8, device="cuda")
        scratch_bytes = int(L.nz_compress_scratch_bytes(n, S))
        scratch = self._scratch_for(scratch_bytes)
        _lib.check(L.nz_compress_bf16(_ptr(flat), n, self.precision, S, _ptr(frac), _ptr(staging),
                                      cap, _ptr(scratch), scratch.numel(), st))
        self._cache[name] = self._finish_write(
            _Entry(n, tensor.dtype, S, 0, staging, frac, normalizers, _next_op()), previous)

    def adamw_update(self, name: str, grad: torch.Tensor, exp_avg: torch.Tensor,
                     exp_avg_sq: torch.Tensor, lr: float, beta1: float, beta2: float, eps: float,
                     weight_decay: float, step: int, grad_scale: float = 1.0) -> bool:
        """The read -> AdamW -> write cycle of one stored weight as a single library call
        (``nz_adamw_compressed_bf16``): the decode kernel applies the step while it produces
        the weights, the compressor codes the result.  Bit for bit what `read`,
        ``nz_adamw_bf16`` and `write` give.  Needs bf16 moments and a bf16 gradient shaped
        like the weight; returns False (nothing done) when the call does not qualify."""
        entry = self._get(name)
        if entry is None:
            raise RuntimeError("Data not found")
        n = entry.numel
        if (self.normalizer_size or entry.normalizers is not None or n % 8
                or any(t.dtype != torch.bfloat16 or not t.is_cuda or t.numel() != n
                       or not t.is_contiguous() or t.data_ptr() % 16
                       for t in (grad, exp_avg, exp_avg_sq))):
            return False
        L, S = self._lib, entry.lane_symbols
        frac = torch.empty_like(entry.fractions)
        cap = int(L.nz_container_bound(n, S))
        staging = torch.empty(cap, dtype=torch.uint8, device="cuda")
        scratch = self._scratch_for(int(L.nz_adamw_compressed_scratch_bytes(n, S)))
        _lib.check(L.nz_adamw_compressed_bf16(
            _ptr(entry.container), entry.container.numel(), _ptr(entry.fractions), n,
            entry.operand_cols, self.precision, S, entry.max_unit_words, int(self.canonical_nan),
            _ptr(grad), _ptr(exp_avg), _ptr(exp_avg_sq), lr, beta1, beta2, eps, weight_decay, step,
            grad_scale, _ptr(frac), _ptr(staging), cap, _ptr(scratch), scratch.numel(),
            _ptr(self._status), _stream()))
        self._cache[name] = self._finish_write(
            _Entry(n, entry.dtype, S, 0, staging, frac, None, _next_op(), entry.operand_cols), entry)
        return True

    # -- settling a write without stalling the host ----------------------------
    def _finish_write(self, entry: _Entry, replaced: Optional[_Entry] = None) -> _Entry:
        """The reference reads the compressed size back right after compressing, which
        blocks the host (cuda/high_level.cu:114-115).  Here the 64-byte container header
        is copied to pinned memory asynchronously; the entry is usable at once (decoding
        from the worst-case-sized buffer) and is right-sized the first time it is touched
        after that copy has completed.  `sync_writes = True` restores the blocking form.
        Header slots (one pinned buffer, 64 bytes each) and events are pooled: a write
        allocates no pinned memory and creates no event once the pools are warm."""
        if replaced is not None and replaced.pending is not None:
            # overwritten before it was ever settled: its slot and event go back (a copy
            # still in flight into the slot lands before the next one, same stream)
            self._release_pending(replaced)
        if not self._hdr_free:
            self._grow_header_pool()
        slot = self._hdr_free.pop()
        event = self._event_pool.pop() if self._event_pool else torch.cuda.Event()
        _lib.check(self._lib.nz_container_header_async(
            _ptr(entry.container), self._hdr_base[slot >> 8] + 64 * (slot & 255), _stream()))
        event.record()
        entry.pending = (slot, event)
        if self.sync_writes:
            self._settle(entry, block=True)
        return entry

    def _grow_header_pool(self) -> None:
        chunk = torch.empty(256 * 64, dtype=torch.uint8).pin_memory()
        index = len(self._hdr_chunks)
        self._hdr_chunks.append(chunk)
        self._hdr_base.append(chunk.data_ptr())
        self._hdr_free.extend(range(256 * index + 255, 256 * index - 1, -1))

    def _release_pending(self, entry: _Entry) -> None:
        slot, event = entry.pending
        self._hdr_free.append(slot)
        self._event_pool.append(event)
        entry.pending = None

    def _settle(self, entry: _Entry, block: bool) -> None:
        if entry.pending is None:
            return
        slot, event = entry.pending
        if block:
            event.synchronize()
        elif not event.query():
            return
        total, words = ctypes.c_uint64(0), ctypes.c_uint32(0)
        rc = self._lib.nz_parse_header(self._hdr_base[slot >> 8] + 64 * (slot & 255),
                                       ctypes.byref(total), ctypes.byref(words))
        self._release_pending(entry)
        if rc:
            raise _lib.NeuzipError("write produced no NZR1 container")
        entry.max_unit_words = words.value
        entry.container = entry.container[:total.value].clone()     # enqueued after the write
        entry.version += 1

    def settle_all(self) -> None:
        """Wait for every write still in flight and right-size its container (for instance
        before capturing decodes in a CUDA graph, where events must not be queried)."""
        for entry in self._cache.values():
            self._settle(entry, block=True)

    def _get(self, name: str) -> Optional[_Entry]:
        entry = self._cache.get(name)
        if entry is not None and entry.pending is not None:
            self._settle(entry, block=False)
        return entry

    def read(self, name: str) -> torch.Tensor:
        """cuda/high_level.cu:223-250 (+ _decompress_and_merge :164-206); no host sync."""
        entry = self._get(name)
        if entry is None:
            raise RuntimeError("Data not found")
        out = torch.empty(entry.numel, dtype=torch.bfloat16, device="cuda")
        self.read_into(name, out)
        return out

    def read_into(self, name: str, out: torch.Tensor) -> None:
        entry = self._get(name)
        if entry is None:
            raise RuntimeError("Data not found")
        # a batch of one: the batched entry point carries the per-item promise that the
        # compressed bytes are not fresh, which lets this launch set up while the previous
        # kernel of the stream drains
        item = (_lib.DecompressItem * 1)()
        item[0].container = _ptr(entry.container)
        item[0].container_bytes = entry.container.numel()
        item[0].frac_in = _ptr(entry.fractions)
        item[0].n = entry.numel
        item[0].max_unit_words = entry.max_unit_words
        item[0].flags = _stable_flag([entry], _next_op())
        item[0].out_bf16 = _ptr(out)
        item[0].operand_cols = entry.operand_cols
        item[0].lane_symbols = entry.lane_symbols
        self._set_normalizer(item[0], entry)
        _lib.check(self._lib.nz_decompress_bf16_batch(
            item, 1, self.precision, entry.lane_symbols, int(self.canonical_nan),
            _ptr(self._status), _stream()))

    def read_rows(self, name: str, rows: torch.Tensor, row_len: int) -> torch.Tensor:
        """Rows ``rows`` (any integer tensor) of the stored tensor seen as a
        ``[numel / row_len, row_len]`` table, as a ``[rows.numel(), row_len]`` bf16 tensor.
        Only the units that hold those rows are decoded (``nz_gather_rows_bf16``);
        nothing synchronises with the host.  Row numbers outside the table raise at
        the next ``check()``.  The reference decompresses the whole
        table for every lookup (neuzip/nn/embedding.py:30-39)."""
        entry = self._get(name)
        if entry is None:
            raise RuntimeError("Data not found")
        if row_len <= 0 or entry.numel % row_len:
            raise ValueError(f"row length {row_len} does not divide the {entry.numel} stored elements")
        rows = rows.reshape(-1).to(device="cuda", dtype=torch.int64)
        k = rows.numel()
        if k == 0:
            return torch.empty(0, row_len, dtype=torch.bfloat16, device="cuda")
        if entry.operand_cols:
            # a matrix in operand order interleaves four rows per block: decode everything
            return self.read(name).view(-1, row_len)[rows]
        U = 32 * entry.lane_symbols
        per_row = 1 if U % row_len == 0 else (row_len // U if row_len % U == 0
                                              else (row_len + U - 1) // U + 1)
        if k * per_row >= (entry.numel + U - 1) // U:
            # the lookups would decode as much as the whole table holds
            return self.read(name).view(-1, row_len)[rows]
        out = torch.empty(k, row_len, dtype=torch.bfloat16, device="cuda")
        L = self._lib
        scratch_bytes = int(L.nz_gather_scratch_bytes(k, row_len, entry.lane_symbols))
        scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device="cuda")
        _lib.check(L.nz_gather_rows_normalized_bf16(
            _ptr(entry.container), entry.container.numel(), _ptr(entry.fractions), entry.numel,
            self.precision, entry.lane_symbols, entry.max_unit_words, int(self.canonical_nan),
            row_len, _ptr(rows), k, _ptr(entry.normalizers),
            self.normalizer_size if entry.normalizers is not None else 0, _ptr(out), _ptr(scratch),
            scratch_bytes, _ptr(self._status), _stream()))
        return out

    def _set_normalizer(self, item, entry: _Entry) -> None:
        """Tensors written with a block normaliser are scaled back by the decoder itself
        (cuda/kernels.cuh:208-216 of the reference does it in its merge kernel)."""
        if entry.normalizers is not None:
            item.normalizers = _ptr(entry.normalizers)
            item.normalizer_group = self.normalizer_size
        else:
            item.normalizers = None
            item.normalizer_group = 0

    def read_many(self, names: Sequence[str]) -> List[torch.Tensor]:
        """Decompress several tensors (for instance all matrices of one layer) with
        as few launches as possible; same results as ``[self.read(n) for n in names]``.
        The reference reads one tensor per call (neuzip/binding.py:88-92); batching lets
        small matrices share the GPU instead of each leaving most SMs idle."""
        entries = []
        for name in names:
            entry = self._get(name)
            if entry is None:
                raise RuntimeError("Data not found")
            entries.append(entry)
        outs = [torch.empty(e.numel, dtype=torch.bfloat16, device="cuda") for e in entries]
        # one batched call; every item names its own lane_symbols
        if entries:
            items = (_lib.DecompressItem * len(entries))()
            flags = _stable_flag(entries, _next_op())
            for k, e in enumerate(entries):
                items[k].container = _ptr(e.container)
                items[k].container_bytes = e.container.numel()
                items[k].frac_in = _ptr(e.fractions)
                items[k].n = e.numel
                items[k].max_unit_words = e.max_unit_words
                items[k].flags = flags
                items[k].out_bf16 = _ptr(outs[k])
                items[k].operand_cols = e.operand_cols
                items[k].lane_symbols = e.lane_symbols
                self._set_normalizer(items[k], e)
            _lib.check(self._lib.nz_decompress_bf16_batch(
                items, len(entries), self.precision, entries[0].lane_symbols,
                int(self.canonical_nan), _ptr(self._status), _stream()))
        return outs

    def make_batch(self, names: Sequence[str], outs: Sequence[torch.Tensor]) -> _Batch:
        """Pre-build the argument block of a batched decode of `names` into the given
        flat bf16 output tensors; returns an object for `run_batch`.  Lets a caller that
        decodes the same tensors again and again (every forward of a layer) skip all
        per-call Python work.  The batch follows the handles, not the bytes: when a
        handle is written again (an optimiser step, a loaded checkpoint) the next
        `run_batch` picks up the new container."""
        batch = _Batch(names, outs)
        self._bind_batch(batch)
        return batch

    def _bind_batch(self, batch: _Batch) -> None:
        entries = [self._cache[n] for n in batch.names]
        for e in entries:
            self._settle(e, block=False)
        # two argument blocks: with and without the promise that the inputs are stable
        blocks = []
        for flags in (0, _lib.NZ_ITEM_INPUTS_STABLE):
            items = (_lib.DecompressItem * len(entries))()
            for k, (e, out) in enumerate(zip(entries, batch.outs)):
                if out.numel() < e.numel or out.dtype != torch.bfloat16 or not out.is_cuda:
                    raise ValueError(
                        "output buffers must be CUDA bf16 tensors of at least numel elements")
                items[k].container = _ptr(e.container)
                items[k].container_bytes = e.container.numel()
                items[k].frac_in = _ptr(e.fractions)
                items[k].n = e.numel
                items[k].max_unit_words = e.max_unit_words
                items[k].flags = flags
                items[k].out_bf16 = _ptr(out)
                items[k].operand_cols = e.operand_cols
                items[k].lane_symbols = e.lane_symbols
                self._set_normalizer(items[k], e)
            blocks.append(items)
        # the entries keep their tensors alive as long as the batch refers to them
        batch.entries, batch.blocks, batch.lane_symbols = entries, blocks, entries[0].lane_symbols
        batch.versions = [e.version for e in entries]

    def run_batch(self, batch: _Batch) -> None:
        cache = self._cache
        for name, entry, version in zip(batch.names, batch.entries, batch.versions):
            # written, imported or erased since -- or its write has settled meanwhile
            if (cache.get(name) is not entry or entry.version != version
                    or (entry.pending is not None and entry.pending[1].query())):
                self._bind_batch(batch)
                break
        items = batch.blocks[1 if _stable_flag(batch.entries, _next_op()) else 0]
        rc = self._lib.nz_decompress_bf16_batch(items, len(batch.names), self.precision,
                                                batch.lane_symbols, int(self.canonical_nan),
                                                _ptr(self._status), _stream())
        if rc:
            _lib.check(rc)

    def size(self, name: str) -> int:
        """cuda/high_level.cu:208-221: stored bytes, 0 for an unknown name."""
        entry = self._cache.get(name)
        if entry is None:
            return 0
        self._settle(entry, block=True)
        extra = 0 if entry.normalizers is None else entry.normalizers.numel()
        return entry.container.numel() + entry.fractions.numel() + extra

    def linear(self, name: str, input: torch.Tensor, shape: Sequence[int],
               bias: torch.Tensor) -> torch.Tensor:
        """cuda/high_level.cu:252-257."""
        fused = self._linear_fused(name, input, shape, bias)
        if fused is None:
            fused = self._linear_vec(name, input, shape, bias)
        if fused is not None:
            return fused
        weight = self.read(name).view(*shape)
        return torch.nn.functional.linear(input, weight, bias)

    def linear_without_bias(self, name: str, input: torch.Tensor,
                            shape: Sequence[int]) -> torch.Tensor:
        """cuda/high_level.cu:259-263."""
        fused = self._linear_fused(name, input, shape, None)
        if fused is None:
            fused = self._linear_vec(name, input, shape, None)
        if fused is not None:
            return fused
        weight = self.read(name).view(*shape)
        return torch.matmul(input, weight.t())

    def linear_allreduce(self, name: str, input: torch.Tensor, shape: Sequence[int],
                         bias: Optional[torch.Tensor], reducer) -> Optional[torch.Tensor]:
        """`all_reduce(input @ W^T) (+ bias on the rank that has it)` for a row-parallel shard,
        the sum over the ranks done by the fused linear kernel's epilogue over peer memory
        (``nz_linear_allreduce_bf16``) instead of a collective after it.  Every rank must
        make the same calls; returns None (on every rank alike: the test only looks at
        shapes, types and the storage order) when the call does not qualify, and the caller
        falls back to `linear` + all-reduce."""
        return self._linear_fused(name, input, shape, bias, reducer)

    def _linear_fused(self, name: str, input: torch.Tensor, shape: Sequence[int],
                      bias: Optional[torch.Tensor], reducer=None) -> Optional[torch.Tensor]:
        """`input @ W^T (+ bias)` with the weight decoded straight into tensor-core operand
        tiles (``nz_linear_bf16``): no bf16 copy of the weight is written or read back.
        Returns None when the call does not qualify (weight not in operand order, input not
        contiguous bf16 on the GPU, more input rows than `fused_linear_max_rows`).  fp32
        accumulation and one rounding to bf16, like the library GEMM; the order of the sums
        differs, so the last bit may."""
        limit = self.fused_linear_max_rows
        if not limit:
            return None
        entry = self._get(name)
        if entry is None or not entry.operand_cols or len(shape) != 2:
            return None
        out_f, in_f = int(shape[0]), int(shape[1])
        if in_f != entry.operand_cols or out_f * in_f != entry.numel:
            return None
        if (input.dtype != torch.bfloat16 or not input.is_cuda or input.dim() < 1
                or input.shape[-1] != in_f):
            return None
        m = input.numel() // in_f
        if m == 0 or m > limit:
            return None
        if bias is not None and (bias.dtype != torch.bfloat16 or not bias.is_cuda
                                 or bias.numel() != out_f):
            return None
        x = input.detach().reshape(m, in_f)
        if not x.is_contiguous() or x.data_ptr() % 16:
            x = x.contiguous()
            if x.data_ptr() % 16:
                return None
        L = self._lib
        y = torch.empty(input.shape[:-1] + (out_f,), dtype=torch.bfloat16, device="cuda")
        if reducer is not None:
            need = int(L.nz_linear_allreduce_workspace_bytes(out_f, in_f, entry.lane_symbols, m,
                                                             reducer.world))
            if not need or not reducer.fits(need):
                return None
            turn, group, before = reducer.next_set()
            after = ctypes.c_uint32(0)
            _next_op()
            rc = L.nz_linear_allreduce_bf16(
                _ptr(entry.container), entry.container.numel(), _ptr(entry.fractions), out_f, in_f,
                self.precision, entry.lane_symbols, entry.max_unit_words, int(self.canonical_nan),
                _ptr(x), m, _ptr(bias.contiguous() if bias is not None else None), _ptr(y),
                ctypes.byref(group), before, ctypes.byref(after), _ptr(self._status), _stream())
            if rc == _lib.NZ_E_CAPACITY:
                # the peers cannot know: a silent fallback here would leave them waiting
                raise RuntimeError("this rank's shard has units too long for the fused linear; "
                                   "switch the fused all-reduce off (fuse_tp_allreduce(None))")
            _lib.check(rc)
            reducer.advance(turn, after.value)
            return y
        need = int(L.nz_linear_workspace_bytes(out_f, in_f, entry.lane_symbols, m))
        if self._lin_ws is None or self._lin_ws.numel() < need:
            self._lin_ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        _next_op()
        rc = L.nz_linear_bf16(
            _ptr(entry.container), entry.container.numel(), _ptr(entry.fractions), out_f, in_f,
            self.precision, entry.lane_symbols, entry.max_unit_words, int(self.canonical_nan),
            _ptr(x), m, _ptr(bias.contiguous() if bias is not None else None), _ptr(y),
            _ptr(self._lin_ws), self._lin_ws.numel(), _ptr(self._status), _stream())
        if rc == _lib.NZ_E_CAPACITY:
            return None          # units too long to sit next to the operand tiles: decode instead
        _lib.check(rc)
        return y

    def _linear_vec(self, name: str, input: torch.Tensor, shape: Sequence[int],
                    bias: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """A single input vector (one token of one sequence, the decode step of
        generation): multiply while decoding instead of writing the bf16 weights out
        and reading them back (``nz_linear_vec_bf16``).  Returns None when the call does
        not qualify; products and sums are fp32 with one rounding to bf16, like the
        library GEMM, but the order of the sums differs, so the last bit may."""
        if not self.fused_vector_linear:
            return None
        entry = self._get(name)
        if (entry is None or entry.normalizers is not None or entry.operand_cols
                or len(shape) != 2):
            return None
        out_f, in_f = int(shape[0]), int(shape[1])
        if (input.dtype != torch.bfloat16 or not input.is_cuda or input.numel() != in_f
                or in_f % 256 or out_f * in_f != entry.numel):
            return None
        if bias is not None and (bias.dtype != torch.bfloat16 or not bias.is_cuda
                                 or bias.numel() != out_f):
            return None
        if torch.is_grad_enabled() and (input.requires_grad or (bias is not None and bias.requires_grad)):
            return None
        L = self._lib
        if self._vec_src is not input or self._vec_ver != input._version:
            # q/k/v and gate/up are called with the same tensor: convert it once
            self._vec_x = input.detach().reshape(-1).float()
            self._vec_src, self._vec_ver = input, input._version
        y = torch.empty(input.shape[:-1] + (out_f,), dtype=torch.bfloat16, device="cuda")
        # partial sums: one buffer per matrix size, reused (calls are ordered on the stream)
        scratch = self._vec_scratch.get((entry.numel, in_f))
        if scratch is None:
            nbytes = int(L.nz_linear_vec_scratch_bytes(entry.numel, in_f, entry.lane_symbols))
            scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
            self._vec_scratch[(entry.numel, in_f)] = scratch
        scratch_bytes = scratch.numel()
        _lib.check(L.nz_linear_vec_bf16(
            _ptr(entry.container), entry.container.numel(), _ptr(entry.fractions), entry.numel,
            self.precision, entry.lane_symbols, entry.max_unit_words, int(self.canonical_nan),
            in_f, _ptr(self._vec_x), _ptr(bias.contiguous() if bias is not None else None),
            _ptr(y), _ptr(scratch), scratch_bytes, _ptr(self._status), _stream()))
        return y

    def split(self, tensor: torch.Tensor) -> List[torch.Tensor]:
        """cuda/high_level.cu:301-321: always full mantissa (f_bits_save = 7, :289);
        returns [exponents, fractions], one byte per element each."""
        _require_bf16(tensor)
        self._ensure_device()
        flat = _as_flat_bf16_cuda(tensor)
        n = flat.numel()
        exp = torch.empty(n, dtype=torch.uint8, device="cuda")
        frac = torch.empty(n, dtype=torch.uint8, device="cuda")
        _lib.check(self._lib.nz_split_bf16(_ptr(flat), n, 7, _ptr(exp), _ptr(frac), _stream()))
        return [exp, frac]

    # -- serialisation ----------------------------------------------------
    def export_entry(self, name: str) -> dict:
        """The stored form of one tensor as CPU tensors plus the numbers needed to
        decode it; what `nn.Linear.get_extra_state` puts into a state_dict."""
        e = self._cache[name]
        self._settle(e, block=True)
        return {"format": "NZR1", "precision": self.precision, "numel": e.numel,
                "lane_symbols": e.lane_symbols, "max_unit_words": e.max_unit_words,
                "container": e.container.cpu(), "fractions": e.fractions.cpu(),
                "normalizer_size": self.normalizer_size,
                "normalizers": None if e.normalizers is None else e.normalizers.cpu(),
                "operand_cols": e.operand_cols}

    def import_entry(self, name: str, blob: dict) -> None:
        """Inverse of `export_entry`: the compressed bytes go straight to the GPU,
        no bf16 copy of the tensor is ever materialised."""
        if (blob.get("format") != "NZR1" or int(blob["precision"]) != self.precision
                or int(blob.get("normalizer_size", 0)) != self.normalizer_size):
            raise ValueError("checkpoint entry does not match this manager "
                             f"(format {blob.get('format')!r}, precision {blob.get('precision')})")
        self._ensure_device()
        container = blob["container"].to(device="cuda", dtype=torch.uint8).contiguous()
        fractions = blob["fractions"].to(device="cuda", dtype=torch.uint8).contiguous()
        n = int(blob["numel"])
        if fractions.numel() != int(self._lib.nz_frac_bytes(n, self.precision)):
            raise ValueError("checkpoint entry: fraction stream has the wrong length")
        normalizers = blob.get("normalizers")
        if normalizers is not None:
            normalizers = normalizers.to(device="cuda", dtype=torch.uint8).contiguous()
        replaced = self._cache.get(name)
        if replaced is not None and replaced.pending is not None:
            self._release_pending(replaced)
        self._cache[name] = _Entry(n, torch.bfloat16, int(blob["lane_symbols"]),
                                   int(blob["max_unit_words"]), container, fractions, normalizers,
                                   _next_op(), int(blob.get("operand_cols", 0)))

    # -- extras -----------------------------------------------------------
    def erase(self, name: str) -> None:
        gone = self._cache.pop(name, None)
        if gone is not None and gone.pending is not None:
            self._release_pending(gone)

    def entry(self, name: str) -> _Entry:
        entry = self._cache[name]
        self._settle(entry, block=True)
        return entry

    def names(self):
        return list(self._cache)


def _make_backend(precision: int, normalizer_size: int):
    cls_name = f"Manager_f{precision}_n{normalizer_size}"
    return type(cls_name, (CodecBackend,), {
        "precision": precision,
        "normalizer_size": normalizer_size,
        "__doc__": f"Backend for precision={precision}, normalizer_size={normalizer_size} "
                   f"(cuda/neuzip.cu:47-105).",
    })


class _CudaNamespace:
    """Attribute access like the extension module: ``_cuda.Manager_f7_n0``."""
    Algorithm = Algorithm

    def __init__(self) -> None:
        for p in PRECISIONS:
            for nsz in NORMALIZER_SIZES:
                cls = _make_backend(p, nsz)
                setattr(self, cls.__name__, cls)


_cuda = _CudaNamespace()
