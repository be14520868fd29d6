"""Multi-GPU partitioning of the decode path (one process per GPU, torch.distributed for the plumbing).

* Decode batches shard by request with no collective: `split_even` / `lpt_assign` decide which rank owns
  which request (each rank keeps its requests' cache pages in its own pool).
* A single long request shards the index-key RANGE: every rank scores all query tokens against its block
  range, emits a local top-k with scores, and the global top-k is re-selected from the ranks' candidates
  (exact: the global top-k is a subset of the union of the local top-ks; ties go to the lower global
  index).  The attention of the request's query tokens is sharded by token slice, so a rank only needs the
  candidates of ITS slice: one all-to-all (`exchange_own_slice`: every rank sends each peer the candidates
  of that peer's tokens, 1/world of what an all-gather would move per link); `sharded_indexer_topk` keeps the
  all-gather form for callers that want the selection of every token on every rank.  The reference indexer
  is single-device (lightning_indexer_quant_impl.py:31-32), so this has no reference counterpart; its result
  equals the unsharded operator's.
"""
from __future__ import annotations

import math
import os
from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist

INT32_MAX = 2 ** 31 - 1


def split_even(n_requests: int, world: int) -> List[List[int]]:
    """Contiguous, as-even-as-possible split of request ids over ranks."""
    base, rem = divmod(n_requests, world)
    out, pos = [], 0
    for r in range(world):
        n = base + (1 if r < rem else 0)
        out.append(list(range(pos, pos + n)))
        pos += n
    return out


def request_cost(ctx_len: int, s1: int = 1, topk: int = 2048) -> float:
    """Relative cost of one request per decode step: the indexer streams 130 B per key, the attention
    gathers 656 B for each of min(ctx, topk) keys per query token."""
    return 130.0 * ctx_len + 656.0 * min(ctx_len, topk) * s1


def lpt_assign(costs: Sequence[float], world: int) -> List[List[int]]:
    """Longest-processing-time-first bin packing of requests onto ranks (ragged production batches)."""
    order = sorted(range(len(costs)), key=lambda i: (-costs[i], i))
    loads = [0.0] * world
    bins: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (loads[j], j))
        bins[r].append(i)
        loads[r] += costs[i]
    for b in bins:
        b.sort()
    return bins


def key_range_for_rank(max_ctx: int, rank: int, world: int, block_size: int = 128):
    """Block-aligned logical key range [begin, end) of `rank`; the last rank takes the remainder."""
    nblk = math.ceil(max_ctx / block_size)
    per = math.ceil(nblk / world)
    begin = min(rank * per, nblk) * block_size
    end = min((rank + 1) * per, nblk) * block_size
    return begin, (INT32_MAX if rank == world - 1 else end)


def token_slice_for_rank(n_tokens: int, rank: int, world: int):
    """Contiguous slice [first, last + 1) of a request's query tokens whose attention `rank` runs."""
    per = math.ceil(n_tokens / world)
    return min(rank * per, n_tokens), min((rank + 1) * per, n_tokens)


def _cuda_local_topk(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq_key, block_table,
                     selected_count, key_begin, key_end):
    from .lightning_indexer_quant_impl import indexer_scores_topk
    t = idx_query.shape[0]
    res = torch.empty((t, 1, selected_count), dtype=torch.int32, device=idx_query.device)
    sc = torch.empty((t, selected_count), dtype=torch.float32, device=idx_query.device)
    indexer_scores_topk(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq_key,
                        block_table, res, selected_count, topk_scores=sc, key_begin=key_begin, key_end=key_end)
    return res.reshape(t, selected_count), sc


def _cuda_merge(cand_scores, cand_ids, k):
    from .lightning_indexer_quant_impl import topk_select
    counts = torch.full((cand_scores.shape[0],), cand_scores.shape[1], dtype=torch.int32, device=cand_scores.device)
    out_idx, _ = topk_select(cand_scores.contiguous(), counts, k, ids=cand_ids.contiguous())
    return out_idx


def sharded_indexer_topk(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq_key,
                         block_table, selected_count: int = 2048, group=None,
                         local_fn: Optional[Callable] = None, merge_fn: Optional[Callable] = None):
    """Key-range-sharded lightning indexer.  Every rank passes the same query-side tensors and a cache that
    holds (at least) its own block range; returns topk indices [t, selected_count] int32 (global logical key
    positions, -1 pads), identical on every rank.

    `local_fn` / `merge_fn` default to the CUDA kernels; the CPU (gloo) tests of the host logic inject
    stand-ins with the same signatures.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    local_fn = local_fn or _cuda_local_topk
    merge_fn = merge_fn or _cuda_merge
    max_ctx = block_table.shape[1] * 128
    begin, end = key_range_for_rank(max_ctx, rank, world)
    idx, sc = local_fn(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq_key, block_table,
                       selected_count, begin, end)
    if world == 1:
        return idx
    # one all-gather of (score, index) candidates: selected_count * 8 bytes per token and rank
    packed = torch.stack([sc.view(torch.int32), idx.to(torch.int32)], dim=0).contiguous()
    gathered = [torch.empty_like(packed) for _ in range(world)]
    dist.all_gather(gathered, packed, group=group)
    cand_sc = torch.cat([g[0].view(torch.float32) for g in gathered], dim=1)
    cand_id = torch.cat([g[1] for g in gathered], dim=1)
    return merge_fn(cand_sc, cand_id, selected_count)


def exchange_own_slice(scores: torch.Tensor, idx: torch.Tensor, group=None, send=None, recv=None):
    """All-to-all of local top-k candidates: `scores` fp32 / `idx` int32 [n_tokens, k] of ALL query tokens over this
    rank's key range go out so that every rank ends up with the candidates of its own token slice
    (`token_slice_for_rank`) from every rank.  Returns (cand_scores fp32, cand_ids int32), each [n_own, world * k],
    rank-major along the second axis.  Token slices are padded to a common length on the wire (pad ids are -1, which
    the merge ignores).  `send` / `recv` are optional reusable int32 buffers [world, 2, per, k]."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n_tokens, k = idx.shape
    per = math.ceil(n_tokens / world)
    t0, t1 = token_slice_for_rank(n_tokens, rank, world)
    if send is None:
        send = torch.empty((world, 2, per, k), dtype=torch.int32, device=idx.device)
    if recv is None:
        recv = torch.empty_like(send)
    full = (n_tokens // per) if per else 0          # peers whose slice is complete
    if full:
        send[:full, 0].copy_(scores[:full * per].view(torch.int32).view(full, per, k))
        send[:full, 1].copy_(idx[:full * per].view(full, per, k))
    if full < world:                                # a ragged last slice, and empty ones after it
        rem = n_tokens - full * per
        send[full:, 1].fill_(-1)
        send[full:, 0].zero_()
        if rem:
            send[full, 0, :rem].copy_(scores[full * per:].view(torch.int32))
            send[full, 1, :rem].copy_(idx[full * per:])
    dist.all_to_all_single(recv.view(-1), send.view(-1), group=group)
    n_own = t1 - t0
    cand_sc = recv[:, 0, :n_own].permute(1, 0, 2).reshape(n_own, world * k).view(torch.float32)
    cand_id = recv[:, 1, :n_own].permute(1, 0, 2).reshape(n_own, world * k)
    return cand_sc, cand_id


def sharded_indexer_topk_own_slice(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq_key,
                                   block_table, selected_count: int = 2048, group=None,
                                   local_fn: Optional[Callable] = None, merge_fn: Optional[Callable] = None):
    """Key-range-sharded lightning indexer for a request whose attention is sharded by query-token slice: every rank
    passes the same query-side tensors and a cache that holds (at least) its own block range, and gets the global
    top-k [n_own, selected_count] int32 of ITS token slice (`token_slice_for_rank`), equal to the rows the
    unsharded operator computes for those tokens."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    local_fn = local_fn or _cuda_local_topk
    merge_fn = merge_fn or _cuda_merge
    max_ctx = block_table.shape[1] * 128
    begin, end = key_range_for_rank(max_ctx, rank, world)
    idx, sc = local_fn(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq_key, block_table,
                       selected_count, begin, end)
    if world == 1:
        return idx
    cand_sc, cand_id = exchange_own_slice(sc, idx.to(torch.int32), group=group)
    if cand_sc.shape[0] == 0:
        return cand_id[:, :selected_count]
    return merge_fn(cand_sc, cand_id, selected_count)


class PeerCandidateBuffers:
    """Candidate buffers of a key-range-sharded indexer that the other ranks of the node write into directly: on every
    rank an int32 and an fp32 array [tokens_per_rank, world, k] in symmetric memory (`torch.distributed._symmetric_memory`:
    the same allocation on every rank, each mapped into every other rank's address space).  The top-k kernel of rank s
    stores the row of token t at [t - owner * tokens_per_rank][s] of the owner's arrays (dsv32_indexer_topk_scatter), so
    after `barrier()` each rank holds world * k candidates for each of its own tokens, already in the layout the merge
    reads.  NCCL-free on the data path: plain stores over NVLink."""

    def __init__(self, n_tokens: int, k: int, device, group=None):
        # Only peer pointers are needed here (plain stores, no multimem): ask torch not to bind the buffers to an NVLink
        # multicast object, which would tie every rank's GPU to the fate of the others.
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("PeerCandidateBuffers: at most 8 ranks (one node)")
        self.k = k
        self.per = math.ceil(n_tokens / self.world)
        self.t0, self.t1 = token_slice_for_rank(n_tokens, self.rank, self.world)
        shape = (self.per, self.world * k)
        self.ids = symm_mem.empty(shape, dtype=torch.int32, device=device)
        self.scores = symm_mem.empty(shape, dtype=torch.float32, device=device)
        self._h_ids = symm_mem.rendezvous(self.ids, group)
        self._h_sc = symm_mem.rendezvous(self.scores, group)
        self.idx_ptrs = [int(p) for p in self._h_ids.buffer_ptrs]
        self.score_ptrs = [int(p) for p in self._h_sc.buffer_ptrs]

    def scatter_arg(self):
        return (self.world, self.rank, self.per, self.idx_ptrs, self.score_ptrs)

    def barrier(self):
        """Every rank's stores have landed once every rank has passed this point in stream order."""
        self._h_ids.barrier()

    def own(self):
        """(cand_scores, cand_ids) [n_own, world * k] of this rank's tokens (views of the symmetric arrays)."""
        n = self.t1 - self.t0
        return self.scores[:n], self.ids[:n]


def sharded_indexer_topk_peer_stores(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq_key,
                                     block_table, buffers: PeerCandidateBuffers, selected_count: int = 2048):
    """`sharded_indexer_topk_own_slice` without a collective: the top-k kernel of every rank writes its candidates
    straight into the owning ranks' buffers (`buffers`, made once), a barrier follows, and the own slice is merged."""
    from .lightning_indexer_quant_impl import indexer_scores_topk
    max_ctx = block_table.shape[1] * 128
    begin, end = key_range_for_rank(max_ctx, buffers.rank, buffers.world)
    buffers.barrier()   # nobody is still merging the previous step's candidates
    indexer_scores_topk(idx_query, idx_query_scale, idx_key_cache, idx_key_scale, idx_weight, act_seq_key, block_table,
                        None, selected_count, key_begin=begin, key_end=end, scatter=buffers.scatter_arg())
    buffers.barrier()
    cand_sc, cand_id = buffers.own()
    if cand_sc.shape[0] == 0:
        return cand_id[:, :selected_count]
    return _cuda_merge(cand_sc, cand_id, selected_count)
