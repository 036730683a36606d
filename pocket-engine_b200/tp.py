"""Tensor-parallel mode for the adapter path (no counterpart in pocket-engine, which is single-GPU).

One process per GPU. A layer is sharded the way its base weights are:

* column-parallel (q, k, v, gate, up): every rank holds the whole A (the shrink is computed redundantly,
  it is cheap) and the rows ``[rank * N/P, (rank + 1) * N/P)`` of B; x is replicated, y is the local column
  slice. No collective.
* row-parallel (o, down): every rank holds the input-column slice ``A[:, rank * K/P : (rank + 1) * K/P]``
  and, of B, only the rows of the output slice it will write; x arrives sharded ``[T, K/P]``. Each rank's
  shrink gives a partial S; the partials are summed over the ranks (NVLink) either by an NCCL all-reduce or by
  the library's own exchange kernel (``connect_exchange`` + ``TPLinear(exchange="fused")``: one launch that
  pushes the partial to every rank, waits for theirs and adds them); then each rank expands its own N/P slice
  of output columns into its partial y (whose reduction afterwards, the base layer's own, therefore receives
  exactly one copy of the adapter term).

Sharding is expressed with the registry's own vocabulary: a shard is just a ``Site`` with the local sizes, a
row-parallel part carrying ``off = rank * N/P`` so the expand lands in the right columns of the full-width
partial y.
"""
import numpy as np

from .sites import Factors, Site, SitePart

COLUMN, ROW = "column", "row"


def shard_site(site, mode, world, rank):
    """The rank's view of a full-size site."""
    parts = []
    off = 0
    for p in site.parts:
        if p.rows % world:
            raise ValueError(f"{p.module}: {p.rows} output features do not split over {world} ranks")
        n = p.rows // world
        if mode == COLUMN:
            parts.append(SitePart(p.module, n, off))  # local y holds only this rank's slices, back to back
            off += n
        else:
            parts.append(SitePart(p.module, n, p.off + rank * n))  # a slice of the full-width partial y
    cols = site.cols
    if mode == ROW:
        if site.cols % (8 * world):
            raise ValueError(f"{site.cols} input features do not split over {world} ranks in multiples of 8")
        cols = site.cols // world
    return Site(site.layer, cols, parts)


def shard_factors(f, site, mode, world, rank):
    """The rank's slice of one module's factors (scale already folded into B)."""
    part = next(p for p in site.parts if p.module == f.module)
    n = part.rows // world
    b = f.b[rank * n:(rank + 1) * n]
    a = f.a
    if mode == ROW:
        k = site.cols // world
        a = f.a[:, rank * k:(rank + 1) * k]
    return Factors(f.layer, f.module, np.ascontiguousarray(a), np.ascontiguousarray(b))


def shard_x(x, mode, world, rank):
    """Row-parallel layers take the rank's input-column slice of x; column-parallel ones all of it."""
    if mode == COLUMN:
        return x
    k = x.shape[1] // world
    return np.ascontiguousarray(x[:, rank * k:(rank + 1) * k])


class ShardedWorkload:
    """A rank's share of a full-size workload (see workloads.config5): sharded sites, factors and inputs.
    ``y_base(si)`` is this rank's base output: its column slice for column-parallel layers, a full-width
    partial (the true base divided evenly over the ranks) for row-parallel ones."""

    def __init__(self, wl, world, rank):
        self.full, self.world, self.rank = wl, world, rank
        self.modes = list(wl.modes)
        self.sites = [shard_site(s, m, world, rank) for s, m in zip(wl.sites, wl.modes)]
        for name in ("ranks", "scale", "row_n", "row_slot", "max_rank", "n_adapters", "tokens", "n_seqs", "seed"):
            setattr(self, name, getattr(wl, name))
        self.name = f"{wl.name}-tp{world}r{rank}"
        self.token_slot, self.cu = wl.token_slot, wl.cu

    def factors(self, i):
        by_module = {p.module: (si, s) for si, s in enumerate(self.full.sites) for p in s.parts}
        out = []
        for f in self.full.factors(i):
            si, site = by_module[f.module]
            out.append(shard_factors(f, site, self.modes[si], self.world, self.rank))
        return out

    def x_bits(self, si):
        return shard_x(self.full.x_bits(si), self.modes[si], self.world, self.rank)

    def y_base(self, si):
        yb = self.full.y_base(si)
        site = self.full.sites[si]
        if self.modes[si] == ROW:
            return (yb / np.float32(self.world)).astype(np.float32)
        cols = []
        for p in site.parts:
            n = p.rows // self.world
            cols.append(yb[:, p.off + self.rank * n:p.off + (self.rank + 1) * n])
        return np.ascontiguousarray(np.concatenate(cols, axis=1))

    def assemble(self, si, outs):
        """The full layer output from every rank's y (list indexed by rank): row-parallel partials add up,
        column-parallel slices interleave back into the parts."""
        site = self.full.sites[si]
        if self.modes[si] == ROW:
            return np.sum(np.stack(outs, 0).astype(np.float64), 0)
        full = np.zeros((len(outs[0]), site.width()), np.float64)  # all rows, or the same sample of rows from every rank
        for r, y in enumerate(outs):
            at = 0
            for p in site.parts:
                n = p.rows // self.world
                full[:, p.off + r * n:p.off + (r + 1) * n] = y[:, at:at + n]
                at += n
        return full


class _DevView:
    """A raw device address as something torch.as_tensor understands (CUDA array interface, f32)."""

    def __init__(self, ptr, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f4", "data": (int(ptr), False),
                                         "version": 2, "strides": None}


def connect_exchange(loras, rank, world, group=None, timeout_ms=2000):
    """Sets up the exchange kernel's peer mappings for one process per GPU: every rank creates its staging
    memory, the 64-byte handles travel through the process group, every rank maps the others'. Ends with a
    barrier so that no rank launches an exchange before all are mapped."""
    import torch.distributed as dist
    loras.exchange_create(world, rank, timeout_ms)
    handles = [None] * world
    dist.all_gather_object(handles, loras.exchange_export(), group=group)
    for p in range(world):
        if p != rank:
            loras.exchange_import(p, handles[p])
    dist.barrier(group=group)


class TPLinear:
    """Linear::forward's adapter bracket for one shard. ``group`` is a torch.distributed process group (NCCL
    on GPUs); for row-parallel layers the shrink's partial sums are summed over the ranks between shrink and
    expand: ``exchange="nccl"`` by an all-reduce on plane 0, ``"fused"`` by the library's one-kernel exchange
    (after connect_exchange)."""

    def __init__(self, loras, site, mode, group=None, base=None, exchange="nccl"):
        import torch
        self.loras, self.site, self.mode, self.group, self.base = loras, site, mode, group, base
        self.exchange = exchange
        self.lora = loras.hook(site)
        # plane 0 of the f32 intermediate as a tensor, for the collective
        self._s = torch.as_tensor(_DevView(loras.s, (loras.max_tokens, loras.lds)), device=f"cuda:{loras.device}") \
            if mode == ROW else None

    def forward(self, x, rows, y, ldy, f32_out=False, lora=None, main=0):
        import torch
        import torch.distributed as dist
        L = self.loras
        if lora is not None:
            L.shrink(self.lora, lora, x, rows, main)
        if self.base is not None:
            self.base(x, rows, y, ldy, f32_out)
        if lora is None:
            return
        if self.mode == ROW and self.exchange == "fused":
            L.s_exchange(self.lora, lora, rows, main)  # K-split partials of every rank -> plane 0, one launch
            L.expand_reduced(self.lora, lora, rows, y, ldy, f32_out, main)
        elif self.mode == ROW:
            L.s_reduce(self.lora, lora, rows, main)  # K-split partials -> plane 0
            dist.all_reduce(self._s[:rows], op=dist.ReduceOp.SUM, group=self.group)
            L.expand_reduced(self.lora, lora, rows, y, ldy, f32_out, main)
        else:
            L.expand(self.lora, lora, rows, y, ldy, f32_out, main)
