"""Multi-GPU driver for the MME path: one process per GPU (torch.distributed), sharding as the path
allows.

* GEMM / batched GEMM / conv forward / dedx have independent output rows: rank r multiplies its block
  of A's rows (its images) by a replica of B (the weights) and writes its block of the output. No
  collective is on the data path.
* dedw reduces over N*H*W: rank r computes a full-size fp32 partial dW from its images, then the
  partials are summed with one all-reduce (NCCL over NVLink on GPUs). The reference's model of this sum
  is the fp32 read-modify-write add of doMemoryWrite (mme/mme_reference/mme_reference_impl.cpp:718-768)
  and the partial-sum compare of its test manager (mme/mme_verification/common/mme_test_manager.cpp:655-690).

The compute itself is always a call into the C ABI on the rank's GPU; this module only plans shards
and issues the collective.
"""
import numpy as np

from . import abi


def shard_range(total, world, rank):
    """Contiguous, balanced [begin, end) of `total` units for `rank` of `world`."""
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_rows_tensor(t, dim, world, rank, elem_size):
    """A view of tensor descriptor `t` restricted to this rank's slice of dimension `dim` (no copy)."""
    begin, end = shard_range(t.sizes[dim], world, rank)
    v = abi.Tensor()
    abi.C.memmove(abi.C.byref(v), abi.C.byref(t), abi.C.sizeof(abi.Tensor))
    v.sizes[dim] = end - begin
    v.data = (t.data or 0) + begin * t.strides[dim] * elem_size
    return v, begin, end


class ShardedCalculator:
    """Runs the calculator's operations data-parallel over the ranks of a torch.distributed group.

    `dist` is torch.distributed (already initialised) or None for a single process. `all_reduce_sum`
    is a callable summing a flat fp32 buffer over ranks in place; by default it wraps dist.all_reduce
    on a torch tensor that aliases the partial dW.
    """

    def __init__(self, calc, dist=None, rank=0, world=1, device=None):
        self.calc, self.dist, self.rank, self.world = calc, dist, rank, world
        self.device = getattr(calc, "device", 0) if device is None else device
        self._shared_b = None

    def host_gemm_shared_b(self, out, x, w, op, cast=None):
        """Host-tensor GEMM of this rank's rows (`x`, `out`: this rank's shards in pinned host memory) by a `w` that is
        the same on every rank. Instead of `world` uploads of the whole of w through the one host, each rank uploads
        1/world of it over PCIe and the ranks all-gather the pieces over NVLink (NCCL); the library then streams the rows
        of x and of the output through the GPU around the resident w."""
        import torch
        calc, world, rank = self.calc, self.world, self.rank
        nbytes = int(np.prod(list(w.sizes))) * abi.ELEM_SIZE[w.dtype]
        piece = ((nbytes + world - 1) // world + 15) // 16 * 16
        if self._shared_b is None or self._shared_b.numel() != piece * world:
            self._shared_b = torch.empty(piece * world, dtype=torch.uint8, device=torch.device("cuda", self.device))
        buf = self._shared_b
        stream = torch.cuda.current_stream(buf.device)
        calc.set_stream(stream.cuda_stream)
        begin = rank * piece
        mine = max(0, min(piece, nbytes - begin))
        if mine:
            calc._check(calc.lib.mmeb200_memcpy_h2d(calc.ctx, buf.data_ptr() + begin, (w.data or 0) + begin, mine))
        if world > 1:
            self.dist.all_gather_into_tensor(buf, buf[begin:begin + piece])
        wd = abi.Tensor()
        abi.C.memmove(abi.C.byref(wd), abi.C.byref(w), abi.C.sizeof(abi.Tensor))
        wd.data, wd.mem_space = buf.data_ptr(), abi.MEM_DEVICE
        try:
            calc.do_batch_gemm(out, x, wd, op, cast)
        finally:
            calc.set_stream(None)

    def batch_gemm_rows(self, out, x, w, op, cast=None):
        """Each rank computes its block of output rows (op ab / abt: rows of x are rows of the output)."""
        assert op in (abi.OP_AB, abi.OP_ABT), "row sharding needs A stored row-major"
        xv, b, e = shard_rows_tensor(x, 1, self.world, self.rank, abi.ELEM_SIZE[x.dtype])
        ov, _, _ = shard_rows_tensor(out, 1, self.world, self.rank, abi.ELEM_SIZE[out.dtype])
        if e > b:
            self.calc.do_batch_gemm(ov, xv, w, op, cast)
        return b, e

    def conv_images(self, out, x, w, y, params, op, rm=abi.RM_NE, cast=None):
        """fwd / dedx: images (the last dim of x and y) are independent."""
        assert op in (abi.OP_FWD, abi.OP_DEDX)
        d = x.dims - 1
        xv, b, e = shard_rows_tensor(x, d, self.world, self.rank, abi.ELEM_SIZE[x.dtype])
        yv, _, _ = shard_rows_tensor(y, d, self.world, self.rank, abi.ELEM_SIZE[y.dtype])
        ov = yv if out is y else (xv if out is x else shard_rows_tensor(out, d, self.world, self.rank, abi.ELEM_SIZE[out.dtype])[0])
        if e > b:
            self.calc.do_convolution(ov, xv, w, yv, params, op, rm, cast)
        return b, e

    def conv_dedw(self, partial, x, w_shape_tensor, y, params, all_reduce_sum):
        """dedw over this rank's images into `partial` (fp32, full dW shape), then one sum over ranks."""
        d = x.dims - 1
        xv, b, e = shard_rows_tensor(x, d, self.world, self.rank, abi.ELEM_SIZE[x.dtype])
        yv, _, _ = shard_rows_tensor(y, d, self.world, self.rank, abi.ELEM_SIZE[y.dtype])
        if e > b:
            self.calc.do_convolution(partial, xv, w_shape_tensor, yv, params, abi.OP_DEDW)
        else:
            self.calc.lib.mmeb200_memset(self.calc.ctx, partial.data, 0, int(np.prod(list(partial.sizes))) * 4)
        if self.world > 1:
            all_reduce_sum()
        return b, e


class PeerExchange:
    """Exchange buffers and flag blocks for the fused dedw exchange (mmeb200_conv_dedw_allreduce), double-buffered.

    Every rank allocates two exchange buffers (mmeb200_peer_exchange_bytes) and two flag blocks, publishes their handles with
    `all_gather_object` (any torch.distributed backend; world == 1 needs none) and opens the peers'.
    `dedw_allreduce` alternates between the two sets, which is what lets ranks drift apart by one step.
    """

    def __init__(self, calc, n_floats, dist=None, rank=0, world=1, deferred_output=False):
        """deferred_output: with a device-resident `out`, the owner's sum and the final copy of an exchange overlap the next
        call's convolution; `out` is then complete after the calculator's next sync()."""
        assert 1 <= world <= 8
        self.calc, self.rank, self.world, self.n = calc, rank, world, n_floats
        self.deferred_output = deferred_output
        self.calls = 0
        mine = []
        for _ in range(2):
            slots, hs = calc.peer_alloc(calc.lib.mmeb200_peer_exchange_bytes(n_floats, world))
            flag, hf = calc.peer_alloc(256)
            mine.append((slots, hs, flag, hf))
        handles = [[(m[1], m[3]) for m in mine]]
        if world > 1:
            gathered = [None] * world
            dist.all_gather_object(gathered, handles[0])
            handles = gathered
        self.opened = []
        self.groups = []
        for b in range(2):
            g = abi.PeerGroup()
            g.rank, g.world, g.step = rank, world, 0
            g.deferred_output = int(deferred_output)
            for j in range(world):
                if j == rank:
                    g.slots[j], g.flags[j] = mine[b][0], mine[b][2]
                else:
                    sp, fp = calc.peer_open(handles[j][b][0]), calc.peer_open(handles[j][b][1])
                    self.opened += [sp, fp]
                    g.slots[j], g.flags[j] = sp, fp
            self.groups.append(g)
        if world > 1:
            dist.barrier()   # nobody starts before every rank has mapped every buffer

    def dedw_allreduce(self, out, x, w, y, params):
        """dW over this rank's images, summed over all ranks into `out` (fp32), asynchronously on the calculator's stream."""
        g = self.groups[self.calls & 1]
        g.step = self.calls >> 1
        self.calc.do_convolution_dedw_allreduce(out, x, w, y, params, g)
        self.calls += 1

    def close(self):
        for ptr in self.opened:
            self.calc.peer_close(ptr)
        self.opened = []
