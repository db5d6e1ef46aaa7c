"""Pose sharding across the GPUs of one node (one process per GPU, ``torch.distributed``).

The Fourier-slice path shards over poses: every slice is independent in projection, and
back-projection is a sum over slices.

* projection: the volume is replicated, each rank projects its own contiguous range of
  poses; no collective is needed (an all-gather is offered for callers that want every
  projection on every rank).
* back-projection: each rank accumulates its slices into its own partial data and weight
  volumes, which live side by side in ONE float32 buffer so that a single NCCL reduce
  (or all-reduce) over NVLink combines both.  A partial volume is final only after the
  rank's last slice -- but the slab-ordered scatter finishes it slab by slab, so the fold and
  the collective of a finished slab overlap the scatter of the following ones
  (``PartialVolumes.add_(final=True)``).

The reference has no multi-GPU layer; this module is new.  The compute callables are
parameters (defaulting to the CUDA operators of this package) so that the host logic --
ranges, buffer layout, collectives -- can be exercised with ``gloo`` on CPU ranks.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def pose_range(num_poses: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Contiguous, balanced [start, stop) range of poses owned by `rank`: the first
    ``num_poses % world_size`` ranks hold one extra pose."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} / world_size {world_size}")
    if num_poses < 0:
        raise ValueError("num_poses must be >= 0")
    base, extra = divmod(num_poses, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def _world(group) -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def project_3d_to_2d_sharded(reconstruction: torch.Tensor, rotations: torch.Tensor,
                             shifts: Optional[torch.Tensor] = None, *, group=None,
                             gather: bool = False, project_fn: Optional[Callable] = None,
                             **kwargs) -> torch.Tensor:
    """Project this rank's range of the GLOBAL pose list.

    rotations [B_rot, P, 3, 3] and shifts [B_s, P, 2] hold all P poses on every rank; the
    volume must already be replicated (e.g. ``dist.broadcast`` once, or built from the
    same seed).  Returns [B, P_local, N, Nh], or with ``gather=True`` the concatenation
    over ranks [B, P, N, Nh] on every rank.
    """
    if project_fn is None:
        from .ops import project_3d_to_2d_forw as project_fn
    rank, world = _world(group)
    if rotations.dim() == 3:
        rotations = rotations.unsqueeze(0)
    if shifts is not None and shifts.dim() == 2:
        shifts = shifts.unsqueeze(0)
    P = rotations.shape[1]
    lo, hi = pose_range(P, rank, world)
    local = project_fn(reconstruction, rotations[:, lo:hi],
                       shifts[:, lo:hi] if shifts is not None else None, **kwargs)
    if not gather or world == 1:
        return local
    # ranks may hold different pose counts: pad to the largest share, gather, trim
    counts = [pose_range(P, r, world)[1] - pose_range(P, r, world)[0] for r in range(world)]
    pmax = max(counts)
    B, _, N, Nh = local.shape
    padded = torch.zeros((B, pmax, N, Nh), dtype=local.dtype, device=local.device)
    padded[:, : hi - lo] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([part[:, :n] for part, n in zip(parts, counts)], dim=1)


_side_streams = {}


def _side_stream(dev: torch.device) -> torch.cuda.Stream:
    """One high-priority stream per device for the fold + collective of finished slabs (their few
    blocks should not queue behind the thousands of the scatter still running)."""
    s = _side_streams.get(dev.index)
    if s is None:
        s = torch.cuda.Stream(device=dev, priority=-1)
        _side_streams[dev.index] = s
    return s


class PartialVolumes:
    """Data (complex64) and weight (float32) volumes of one rank, adjacent in one float32
    buffer: [ data.re/im interleaved | weights ], so one collective reduces both.

    ``add_`` accumulates a chunk of slices.  On a CUDA device, weighted slices go through a
    persistent interleaved accumulator (16-byte (re, im, weight, 0) voxels, one vector reduction
    per tap, nothing zero-filled or folded per chunk); ``flush`` folds it into ``data`` /
    ``weights``, which are therefore complete only after ``flush()`` (``reduce`` calls it).

    Overlapping the tail: the LAST chunk(s) of a rank can be given with ``final=True``.  They are
    kept (not launched) until ``flush`` / ``reduce``, which then scatters them slab by slab: the
    accumulator's planes are cut into slabs, a slab's planes are final once its pass over the
    final chunks has run, and while later slabs are still being scattered the finished ones are
    folded -- and, in ``reduce``, handed to the collective -- on a second stream."""

    def __init__(self, batch: int, box: int, device, with_weights: bool = True):
        self.shape = (batch, box, box, box // 2 + 1)
        n = batch * box * box * (box // 2 + 1)
        self.flat = torch.zeros(n * (3 if with_weights else 2), dtype=torch.float32, device=device)
        self.data = torch.view_as_complex(self.flat[: 2 * n].view(*self.shape, 2))
        self.weights = self.flat[2 * n:].view(self.shape) if with_weights else None
        self._accum = None          # interleaved accumulator, made on first use
        self._pending = False       # sums in _accum not yet folded into data / weights
        self._stale = False         # _accum still holds sums that were folded already: clear before reuse
        self._flat_zero = True      # data / weights have not been written yet (a fold may overwrite them)
        self._final = []            # chunks kept for the slab-by-slab final stage
        self.slab_groups = 12       # launches the final stage is cut into (each followed by a fold [+ collective])
        self.timing = False         # record last_scatter_done as a timing event (for benchmarks)
        self.last_scatter_done = None   # event after the last scatter launch of the latest final stage

    def _accumulator(self):
        from . import ops
        if self._accum is None:
            self._accum = ops.new_backprojection_accumulator(self.shape[0], self.shape[1], self.flat.device)
        elif self._stale:
            self._accum.zero_()
        self._stale = False
        return self._accum

    def add_(self, projections: torch.Tensor, rotations: torch.Tensor,
             weights: Optional[torch.Tensor] = None, shifts: Optional[torch.Tensor] = None, *,
             interpolation: str = "linear", oversampling: float = 1.0,
             fourier_radius_cutoff: Optional[float] = None, final: bool = False) -> None:
        """Back-project one chunk of device-resident slices [B, P, N, Nh] into these volumes.
        ``final=True``: this chunk belongs to the rank's last ones; it is kept and scattered slab
        by slab inside ``flush`` / ``reduce`` (the tensors must stay unchanged until then)."""
        from . import ops
        kw = dict(interpolation=interpolation, oversampling=oversampling, fourier_radius_cutoff=fourier_radius_cutoff)
        if weights is not None and self.weights is not None and projections.dtype == torch.complex64:
            if final and projections.is_cuda:
                call = ops.prepare_accumulate_interleaved(self._accumulator(), projections, rotations, weights, shifts, **kw)
                if call is not None:
                    self._final.append(call)
            else:
                ops.backproject_2d_to_3d_accumulate_interleaved_(self._accumulator(), projections, rotations, weights, shifts, **kw)
            self._pending = True
        else:
            ops.backproject_2d_to_3d_accumulate_(self.data, self.weights, projections, rotations, weights, shifts, **kw)
            self._flat_zero = False

    def _ranges(self, parts: int):
        n = self.data.numel()
        step = -(-n // max(1, parts))
        return [(lo, min(n, lo + step)) for lo in range(0, n, step)]

    def _fold(self, first: int, stop: int) -> None:
        from . import ops
        ops.fold_backprojection_accumulator(self._accum, self.data, self.weights, accumulate=not self._flat_zero,
                                            voxel_range=(first, stop))

    def _folded(self) -> None:
        self._pending = False
        self._stale = True          # cleared lazily, by the next add_ (a rank that reduces once never pays for it)
        self._flat_zero = False

    def _finish_by_slabs(self, after_part: Optional[Callable]) -> None:
        """Scatter the kept final chunks slab group by slab group on the current stream; fold (and
        report) the voxels of each finished group on the side stream meanwhile."""
        from . import _abi
        dev = self.flat.device
        B, R = self.shape[0], self.shape[1]
        per_item = R * R * (R // 2 + 1)
        slabs, _ = _abi.accumulator_slab_plan(R)
        group = max(1, -(-slabs // max(1, self.slab_groups)))
        main = torch.cuda.current_stream(dev)
        side = _side_stream(dev)
        side.wait_stream(main)                  # everything added so far precedes the folds
        for g0 in range(0, slabs, group):
            n = min(group, slabs - g0)
            for call in self._final:
                _abi.backproject_accumulate_slabs(*call, g0, n)
            done = torch.cuda.Event(enable_timing=self.timing)
            done.record(main)
            self.last_scatter_done = done
            side.wait_event(done)
            with torch.cuda.stream(side):
                for b in range(B):
                    for first, stop in _abi.accumulator_slab_voxels(R, g0, n):
                        self._fold(b * per_item + first, b * per_item + stop)
                        if after_part is not None:
                            after_part(b * per_item + first, b * per_item + stop)
        main.wait_stream(side)
        self._final = []

    def flush(self, parts: int = 1, after_part: Optional[Callable] = None) -> None:
        """Fold the interleaved accumulator (if it holds anything) into data / weights;
        ``after_part(first, stop)`` is called once a range of voxels is complete.  Without kept
        final chunks the volume is folded in `parts` ranges (with nothing pending, after_part is
        just called once per range); with them, slab group by slab group (see the class text), and
        after_part runs with the side stream current."""
        if self._final:
            self._finish_by_slabs(after_part)
            self._folded()
            return
        for first, stop in self._ranges(parts):
            if self._pending:
                self._fold(first, stop)
            if after_part is not None:
                after_part(first, stop)
        if self._pending:
            self._folded()

    def reduce(self, dst: Optional[int] = 0, group=None, parts: int = 4) -> None:
        """Sum the partial volumes over ranks: onto rank `dst`, or onto every rank when dst is
        None.  The volumes are handled in ranges: the collective of a range (data and weights of
        the same voxels) starts as soon as that range is complete, while the next range is folded
        -- or, with final chunks kept by ``add_(final=True)``, still being scattered.  Outside an
        initialised process group only the pending sums are folded."""
        _, world = _world(group)
        if world == 1:
            self.flush()
            return
        n = self.data.numel()
        works = []

        def start(first: int, stop: int) -> None:
            pieces = [self.flat[2 * first: 2 * stop]]
            if self.weights is not None:
                pieces.append(self.flat[2 * n + first: 2 * n + stop])
            for piece in pieces:
                if dst is None:
                    works.append(dist.all_reduce(piece, op=dist.ReduceOp.SUM, group=group, async_op=True))
                else:
                    works.append(dist.reduce(piece, dst=dst, op=dist.ReduceOp.SUM, group=group, async_op=True))

        self.flush(parts=parts if self._pending else 1, after_part=start)
        for w in works:
            w.wait()


def backproject_2d_to_3d_sharded(projections: torch.Tensor, rotations: torch.Tensor,
                                 weights: Optional[torch.Tensor] = None,
                                 shifts: Optional[torch.Tensor] = None, *,
                                 interpolation: str = "linear", oversampling: float = 1.0,
                                 fourier_radius_cutoff: Optional[float] = None,
                                 chunk: int = 8192, dst: Optional[int] = 0, group=None,
                                 into: Optional[PartialVolumes] = None, reduce: bool = True,
                                 overlap_tail: bool = True,
                                 accumulate_fn: Optional[Callable] = None,
                                 rec_boxsize_fn: Optional[Callable] = None) -> PartialVolumes:
    """Back-project this rank's LOCAL slices [B, P_local, N, Nh] into its partial volumes
    in chunks of `chunk` poses, then (``reduce=True``) combine the ranks' partial volumes
    with one reduce.  Pass ``into=`` to keep accumulating into existing partial volumes
    over several calls and ``reduce=False`` to postpone the collective to the last call
    (the volumes are complete after ``reduce()`` or ``flush()``).  With ``overlap_tail`` (and
    ``reduce``) the last chunk -- together with the one before it when it is shorter than half a
    chunk -- is scattered slab by slab so that the fold and the collective of finished slabs
    overlap it (``PartialVolumes.add_(final=True)``).
    """
    use_add = accumulate_fn is None           # the package's own CUDA path
    if rec_boxsize_fn is None:
        from ._abi import rec_boxsize as rec_boxsize_fn
    if projections.dim() != 4:
        raise ValueError("Projections must be a 4D tensor (B, P, height, width/2+1)")
    if rotations.dim() == 3:
        rotations = rotations.unsqueeze(0)
    if shifts is not None and shifts.dim() == 2:
        shifts = shifts.unsqueeze(0)
    B, P, N, _ = projections.shape
    vols = into
    if vols is None:
        vols = PartialVolumes(B, rec_boxsize_fn(N, oversampling), projections.device,
                              with_weights=weights is not None)
    chunk = max(1, chunk)
    spans = [(lo, min(P, lo + chunk)) for lo in range(0, P, chunk)]
    tail = use_add and reduce and overlap_tail and weights is not None and projections.is_cuda
    if tail and len(spans) >= 2 and spans[-1][1] - spans[-1][0] < chunk // 2:
        spans[-2:] = [(spans[-2][0], spans[-1][1])]          # a short last chunk joins the one before it
    for k, (lo, hi) in enumerate(spans):
        chunk_args = (projections[:, lo:hi], rotations[:, lo:hi],
                      weights[:, lo:hi] if weights is not None else None,
                      shifts[:, lo:hi] if shifts is not None else None)
        kw = dict(interpolation=interpolation, oversampling=oversampling, fourier_radius_cutoff=fourier_radius_cutoff)
        if use_add:
            vols.add_(*chunk_args, final=tail and k == len(spans) - 1, **kw)
        else:
            accumulate_fn(vols.data, vols.weights, *chunk_args, **kw)
    if reduce:
        vols.reduce(dst=dst, group=group)
    return vols
