"""Vocab-parallel sampling across the GPUs of one node: each rank holds V/N columns of every row.

The driver below owns the SEQUENCE of stages and collectives; the per-shard arithmetic is done by a
`compute` object -- the CUDA kernels behind ``rs_vp_stage`` (default), or any object with the same
``stage(name, round)`` method operating on the same workspace regions (the CPU test-suite plugs a numpy
model in and runs the driver over gloo).

Fast protocol (default): 2 all-reduces + 1 all-gather.  Every shard extracts a short candidate list (elements above
a bound read off an all-reduced octave histogram of the row), the lists are all-gathered and every rank finishes the row on the union
from identical data -- no id exchange.  If some row's list cannot settle its cutoff (flagged on the device, read by
the host) the call is repeated with the staged protocol: 13 small collectives:

    MAX(row maxima) . SUM(denominators) . 8 x SUM(counts and masses at 15 pivots) . SUM(threshold tallies) .
    SUM(kept weight per shard) . MAX(sampled id + 1)

Every rank derives the same search bracket, the same owner shard and the same id from the same reduced
numbers; nothing but those numbers crosses the links.  The reference has no multi-GPU mode (no collective
anywhere in sampling.cu); the semantics are those of its kernels on the union of the shards.
"""
import ctypes as C

import torch
import torch.distributed as dist

from . import abi

STAGES = {"max": 0, "sum": 1, "round": 2, "tally": 3, "weight": 4, "pick": 5, "penalty": 6,
          "f_max": 10, "f_sum": 11, "f_compact": 12, "f_finish": 13, "f_advance": 14, "f_extract": 15}


class CudaCompute:
    """Runs the stages with the library's kernels on the current CUDA device."""

    def __init__(self):
        self.L = abi.load()
        self.call = abi.VpCall()

    def bind(self, s, logits, states, penalties, temperature, top_k, top_p, presence, repetition, decay):
        c = self.call
        c.logits, c.states, c.workspace = logits.data_ptr(), states.data_ptr(), s.ws.data_ptr()
        c.penalties = penalties.data_ptr() if penalties is not None else None
        c.stream = torch.cuda.current_stream().cuda_stream
        c.B, c.T, c.V_local, c.V_global, c.col0 = s.B, s.T, s.V_local, s.V_global, s.col0
        c.top_k, c.temperature, c.top_p = top_k, temperature, top_p
        c.presence_penalty, c.repetition_penalty, c.penalty_decay = presence, repetition, decay
        c.rank, c.world = s.rank, s.world

    def tile_begin(self):
        rc = self.L.rs_vp_tile_begin(C.byref(self.call))
        if rc != 0:
            raise RuntimeError(abi.status_string(rc))

    def tile_max(self, tile, col_begin):
        """tile: (B, ncols) fp32 view (last dimension contiguous) of local columns [col_begin, col_begin + ncols)."""
        rc = self.L.rs_vp_tile_max(C.byref(self.call), tile.data_ptr(), tile.stride(0), col_begin, tile.shape[1])
        if rc != 0:
            raise RuntimeError(abi.status_string(rc))

    def stage(self, name, rnd=0):
        rc = self.L.rs_vp_stage(C.byref(self.call), STAGES[name], rnd)
        if rc != 0:
            if rc in (abi.RS_ERR_VOCAB, abi.RS_ERR_BATCH, abi.RS_ERR_TEMPERATURE):
                raise ValueError(abi.status_string(rc))
            raise RuntimeError(abi.status_string(rc))


class VocabParallelSampler:
    def __init__(self, B, V_global, rank, world, group=None, device="cuda", compute=None, T=1, fast=True, graph=False,
                 defer_check=False):
        if V_global % world or (V_global // world) % 4:
            raise ValueError("V=%d cannot be split into %d shards of a multiple of 4 columns" % (V_global, world))
        self.B, self.T, self.V_global, self.rank, self.world, self.group = B, T, V_global, rank, world, group
        self.V_local = V_global // world
        self.col0 = rank * self.V_local
        L = abi.load()
        off = (C.c_int64 * 6)()
        L.rs_vp_layout(B, world, off)
        n = L.rs_vp_workspace_bytes(B, world) // 4
        self.ws = torch.zeros(n, dtype=torch.float32, device=device)
        o = [int(x) for x in off]
        R, P = abi.VP_ROUNDS, 15
        self.gmax = self.ws[o[0]:o[0] + B]
        self.gsum = self.ws[o[1]:o[1] + B]
        self.tallies = [self.ws[o[2] + r * B * P * 2:o[2] + (r + 1) * B * P * 2] for r in range(R)]
        self.gtally = self.ws[o[3]:o[3] + B * 4]
        self.weights = self.ws[o[4]:o[4] + B * world]
        self.ids = self.ws[o[5]:o[5] + B].view(torch.int32)
        self.compute = compute or CudaCompute()
        # fast protocol (3 collectives): regions behind the staged protocol's
        self.fast = fast
        fo = (C.c_int64 * 11)()
        L.rs_vp_fast_layout(B, self.V_local, world, fo)
        f = [int(x) for x in fo]
        S, Lmax = f[8], f[9]
        if world * S > 64:     # the fast protocol's finishing kernel holds 64 segments per row: larger groups run the staged one
            self.fast = False
        self.f_stat1 = self.ws[f[0]:f[0] + B * S]
        self.f_stat2 = self.ws[f[1]:f[1] + B * S * f[10]]
        self.f_send = self.ws[f[2]:f[2] + B * Lmax * 2]
        self.f_send_cnt = self.ws[f[3]:f[3] + B * S]          # one count per (row, sub-block) segment
        # lists and counts lie back to back and travel as ONE block in one all-gather; rank r's block lands r blocks on
        block = f[4] - f[2]
        self.f_send_block = self.ws[f[2]:f[2] + block]
        self.f_gath_block = self.ws[f[4]:f[4] + world * block]
        per_rank = self.f_gath_block.view(world, block)
        self.f_gath = per_rank[:, :B * Lmax * 2]              # (world, B * Lmax * 2) view
        self.f_gath_cnt = per_rank[:, f[3] - f[2]:f[3] - f[2] + B * S]
        self.f_ids = self.ws[f[6]:f[6] + B].view(torch.int32)
        self.f_valid = self.ws[f[7]:f[7] + B].view(torch.int32)
        self.f_all_valid = self.ws[f[7] + B:f[7] + B + 1].view(torch.int32)   # cleared if any row could not be settled
        self.use_graph = graph and fast
        self._graphs = {}
        self.last_protocol = None
        # defer_check: `sample()` does not wait for the device's validity flag; call `validate()` before trusting the
        # ids of the last call (a decode loop does so when it reads the ids on the host)
        self.defer_check = defer_check
        self._pending = None
        self._max_from_tiles = False

    def release_graphs(self):
        """Drops the recorded CUDA graphs.  Call it before the process group is destroyed (and before the process
        exits): NCCL waits for every graph that captured its collectives to be gone before a communicator shuts down."""
        self._graphs.clear()
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def _reduce(self, t, op):
        if self.world > 1:
            dist.all_reduce(t, op=op, group=self.group)

    def _gather(self, out, inp):
        if self.world > 1:
            dist.all_gather_into_tensor(out, inp, group=self.group)
        else:
            out.copy_(inp)

    def begin_tiles(self, logits, states, temperature, top_k, top_p, penalties=None, presence_penalty=0.0,
                    repetition_penalty=0.0, penalty_decay=0.0):
        """lm_head epilogue hook: call before the producer hands over the first tile of this step's logits; then
        `push_tile(tile, col_begin)` per tile as it is produced (any order), then `sample(..., max_from_tiles=True)` with
        the same arguments.  `logits` is the buffer the tiles end up in (the later stages read it)."""
        self._tile_args = (logits, states, penalties, float(temperature), int(top_k), float(top_p), float(presence_penalty),
                           float(repetition_penalty), float(penalty_decay))
        self.compute.bind(self, *self._tile_args)
        self.compute.tile_begin()

    def push_tile(self, tile, col_begin):
        self.compute.tile_max(tile, col_begin)

    def _fast_stages(self, penalties):
        """The device side of the fast protocol: four kernels, four collectives, then the state advance and the penalty
        update, which the device applies only if every row was settled."""
        c = self.compute
        if not self._max_from_tiles:
            c.stage("f_max")
        self._reduce(self.f_stat1, dist.ReduceOp.MAX)
        c.stage("f_sum")
        self._reduce(self.f_stat2, dist.ReduceOp.SUM)
        c.stage("f_extract")
        c.stage("f_compact")
        self._gather(self.f_gath_block, self.f_send_block)
        c.stage("f_finish")
        c.stage("f_advance")
        if penalties is not None:
            c.stage("penalty", 1)

    def _sample_fast(self, bind_args, penalties):
        """Returns ids, or None when some row's candidate list could not settle its cutoff.  With `graph=True` the
        second call with the same buffers and parameters records the stages into a CUDA graph, later ones replay it."""
        if self.use_graph:
            key = (bind_args[0].data_ptr(), bind_args[1].data_ptr(), penalties.data_ptr() if penalties is not None else 0) + \
                tuple(bind_args[3:])
            g = self._graphs.get(key)
            if g is None:
                self.compute.bind(self, *bind_args)
                self._fast_stages(penalties)            # eager the first time (communicators, kernel attributes)
                self._graphs[key] = False
            elif g is False:
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self.compute.bind(self, *bind_args)  # picks up the capture stream
                    self._fast_stages(penalties)
                self._graphs[key] = g
                g.replay()
            else:
                g.replay()
        else:
            self._fast_stages(penalties)
        if self.defer_check:
            # No host synchronisation: the ids are returned as they are.  The device has already withheld the state
            # advance and the penalty update if some row could not be settled; `validate()` finds out and repeats.
            self._pending = (bind_args, penalties)
            return self.f_ids - 1
        if int(self.f_all_valid.item()) == 0:            # the one host synchronisation of the fast protocol
            return None
        return self.f_ids - 1

    def validate(self):
        """After `sample()` calls made with `defer_check=True`: reads the device's verdict on the LAST call (one host
        synchronisation, typically the one the caller needs anyway to read the ids).  If some row's candidate list
        could not settle its cutoff, that call changed nothing on the device; it is repeated here with the staged
        protocol and the corrected ids are returned.  Otherwise returns None: the ids already returned stand."""
        if self._pending is None:
            return None
        bind_args, penalties = self._pending
        self._pending = None
        if int(self.f_all_valid.item()) != 0:
            return None
        self.compute.bind(self, *bind_args)
        return self._sample_staged(penalties)

    def sample(self, logits, states, temperature, top_k, top_p, penalties=None, presence_penalty=0.0,
               repetition_penalty=0.0, penalty_decay=0.0, max_from_tiles=False):
        """logits: this rank's (B, V_local) or (B, T, V_local) fp32 shard; states: replica of setup_rand(seed, B).
        Returns int32 (B,) global token ids, identical on every rank; states / penalties updated in place."""
        assert logits.shape[-1] == self.V_local and logits.dtype == torch.float32
        assert (logits.shape[1] if logits.dim() == 3 else 1) == self.T
        c = self.compute
        bind_args = (logits, states, penalties, float(temperature), int(top_k), float(top_p), float(presence_penalty),
                     float(repetition_penalty), float(penalty_decay))
        c.bind(self, *bind_args)
        self.last_protocol = "staged"
        self._max_from_tiles = bool(max_from_tiles) and self.fast and not self.use_graph
        if self.fast:
            ids = self._sample_fast(bind_args, penalties)
            if ids is not None:
                self.last_protocol = "fast"
                return ids
        return self._sample_staged(penalties)

    def _sample_staged(self, penalties):
        c = self.compute
        self.last_protocol = "staged"
        c.stage("max")
        self._reduce(self.gmax, dist.ReduceOp.MAX)
        c.stage("sum")
        self._reduce(self.gsum, dist.ReduceOp.SUM)
        for r in range(abi.VP_ROUNDS):
            c.stage("round", r)
            self._reduce(self.tallies[r], dist.ReduceOp.SUM)
        c.stage("tally")
        self._reduce(self.gtally, dist.ReduceOp.SUM)
        c.stage("weight")
        self._reduce(self.weights, dist.ReduceOp.SUM)
        c.stage("pick")
        self._reduce(self.ids, dist.ReduceOp.MAX)
        if penalties is not None:
            c.stage("penalty")
        return self.ids - 1
