"""Split-KV decode attention across the GPUs of one node.

The reference is single-device; this is the one multi-GPU step the path has.  The KV sequence of
every kv head is cut into `world` contiguous slices, rank r keeping rows
[bounds[r], bounds[r+1]) in its own HBM.  A decode step is
    local partial (m, l, O) over the slice       the split kernel
    exchange of the world records                 [n_head][head_dim + 4] fp32 = {O, m, l, 0, 0} per rank
    log-sum-exp merge on every rank
The exchange is latency-bound (8448 bytes per rank for 16 heads of 128).  Two forms:
    PeerSplitKVDecoder   a small launch behind the decode launch (one CTA per head) stores the record into every rank's
                         exchange buffer over NVLink (peer stores, every value tagged with the call's generation) and
                         waits for the others' records in its own buffer: no collective call, two launches per layer
                         call, graph-capturable
    SplitKVDecoder       oattn_decode_partial -> NCCL all-gather (torch.distributed) -> oattn_combine

The slicing and the gather are plain host logic that also runs on CPU tensors with the gloo
backend (that is how they are tested without GPUs); the kernels are reached only through
orin_llm_b200.ops and have no CPU counterpart.
"""
import torch
import torch.distributed as dist

PART_PAD = 4
TILE = 64   # slices start on a multiple of the decode kernel's tile


def slice_bounds(n_rows, world):
    """Contiguous, tile-aligned, near-equal slices of [0, n_rows): returns world+1 boundaries."""
    n_tiles = (n_rows + TILE - 1) // TILE
    bounds = [min(n_rows, ((r * n_tiles) // world) * TILE) for r in range(world)]
    bounds.append(n_rows)
    return bounds


def gather_records(local, world_buf, group=None):
    """All-gather one record per rank.  local: [n_head][hd+4]; world_buf: [world][n_head][hd+4]."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world_buf.dim() != local.dim() + 1 or world_buf.shape[0] != world or tuple(world_buf.shape[1:]) != tuple(local.shape):
        raise ValueError("gather_records: buffer of shape %s does not hold %d records of shape %s" % (
            tuple(world_buf.shape), world, tuple(local.shape)))
    if world == 1:
        world_buf[0].copy_(local)
        return world_buf
    if local.is_cuda:
        dist.all_gather_into_tensor(world_buf, local, group=group)
    else:   # gloo: list form
        chunks = [world_buf[r] for r in range(world)]
        dist.all_gather(chunks, local, group=group)
    return world_buf


class PeerSplitKVDecoder:
    """Split-KV decode whose record exchange is done by a kernel of this library: a launch of one CTA per head behind the
    decode launch merges the group results that launch left for its kv head into the rank's record and stores it into every
    rank's exchange buffer with plain peer stores over NVLink (every
    value tagged with the call's generation number), then waits (bounded) until the other ranks' values of this
    generation have arrived in its own buffer and writes the merged output.  Two launches per layer call, no collective
    call, graph-capturable; fused=False keeps the wait in a launch of its own.
    The exchange buffers come from torch's symmetric memory (CUDA VMM mappings of every rank's block).  torch would also
    bind such a block to an NVLink multicast object where the hardware has one; TORCH_SYMM_MEM_DISABLE_MULTICAST=1 is set
    here (unless the caller set it) so that none is created: the kernels use plain peer stores only, and a rank must
    never exit while bound to a multicast object.  No library kernel ever sees a peer pointer."""

    def __init__(self, n_head, n_kv, head_dim, group=None, fused=True):
        import os
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        from . import ops
        self.ops = ops
        self.fused = fused
        self.n_head, self.n_kv, self.head_dim = n_head, n_kv, head_dim
        group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        nbytes = ops.peer_buffer_bytes(self.world, n_head, head_dim)
        if nbytes == 0:
            raise RuntimeError("peer exchange does not cover this shape / world size")
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group)
        self.peer_bufs_dev = int(self.handle.buffer_ptrs_dev)
        self.state = torch.zeros(ops.peer_state_bytes(n_head), dtype=torch.uint8, device="cuda")
        self.workspace = ops.decode_workspace(n_head, n_kv, head_dim)
        torch.cuda.synchronize()
        dist.barrier(group)            # every buffer is zeroed before anyone stores into it

    def decode(self, q, kc_local, vc_local, n_ctx_local, d_len_local, scale, out):
        o = self.ops
        if self.fused:
            o.attn_decode_peer(q, kc_local, vc_local, out, self.n_head, self.n_kv, self.head_dim, n_ctx_local, d_len_local,
                               scale, self.peer_bufs_dev, self.rank, self.world, self.state, self.workspace)
            return out
        o.attn_decode_partial_push(q, kc_local, vc_local, self.n_head, self.n_kv, self.head_dim, n_ctx_local, d_len_local,
                                   scale, self.peer_bufs_dev, self.rank, self.world, self.state, self.workspace)
        o.attn_peer_wait_combine(self.buf, self.world, out, self.n_head, self.head_dim, self.state)
        return out

    def decode_fused(self, q, k_new, v_new, kc_local, vc_local, n_ctx_local, d_len_local, d_pos, scale, rope, out, fuse=None):
        """Decode step with the fused prologue: q unrotated on every rank; the rank that holds the newest rows (the
        last one) passes k_new / v_new, which are rotated at the global position *d_pos and appended at local row
        *d_len_local - 1; the other ranks pass None."""
        o = self.ops
        if fuse is None:
            fuse = o.FUSE_ALL if k_new is not None else o.FUSE_ROPE_Q
        o.attn_decode_peer_fused(q, k_new, v_new, kc_local, vc_local, out, self.n_head, self.n_kv, self.head_dim, n_ctx_local,
                                 d_len_local, d_pos, scale, fuse, rope, self.peer_bufs_dev, self.rank, self.world, self.state,
                                 self.workspace)
        return out

    def status(self):
        return self.ops.peer_status(self.state, self.n_head)


class SplitKVDecoder:
    """Decode attention over a KV sequence that is sharded by rows across the ranks of `group`."""

    def __init__(self, n_head, n_kv, head_dim, group=None):
        from . import ops
        self.ops = ops
        self.n_head, self.n_kv, self.head_dim = n_head, n_kv, head_dim
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        rec = head_dim + PART_PAD
        self.local = torch.zeros(n_head, rec, device="cuda")
        self.parts = torch.zeros(self.world, n_head, rec, device="cuda")
        self.workspace = ops.decode_workspace(n_head, n_kv, head_dim)

    def decode(self, q, kc_local, vc_local, n_ctx_local, d_len_local, scale, out):
        """q [n_head][hd] (replicated); kc/vc_local [n_kv][n_ctx_local][hd] fp16 holding this rank's rows;
        d_len_local: device int32 scalar, valid local rows.  out [n_head][hd] is written on every rank."""
        o = self.ops
        if self.world == 1:
            # no exchange: the split kernel's partials go straight through the in-launch combine
            o.attn_decode_partial(q, kc_local, vc_local, self.parts[0], self.n_head, self.n_kv, self.head_dim,
                                  n_ctx_local, d_len_local, scale, self.workspace)
        else:
            o.attn_decode_partial(q, kc_local, vc_local, self.local, self.n_head, self.n_kv, self.head_dim,
                                  n_ctx_local, d_len_local, scale, self.workspace)
            gather_records(self.local, self.parts, self.group)
        o.attn_combine(self.parts, self.world, out, self.n_head, self.head_dim)
        return out
