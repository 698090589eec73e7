"""FP8 delayed-scaling surface: DelayedScaling recipe, per-layer meta tensors, the
once-per-step amax -> scale update and the Dense forward built on Fp8Quantize / Fp8Matmul.

Mirrors itex/python/fp8/recipe.py:30-93 (DelayedScaling), itex/python/fp8/autocast.py:44-121
(amax_and_scale_update) and the forward half of itex/python/transformer/base.py:48-93 and
layer.py:65-100,170-194 (meta layout: slot 0 = input, 1 = weight, 2 = output per GEMM).
State lives in three device tensors per direction, updated by one small kernel
(itexb_fp8_amax_and_scale_update) instead of a chain of TF ops.
"""
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Optional

import torch

from . import kernels as K
from . import ops

FP8_MAX_FWD = 448.0     # e4m3 (Format.HYBRID max_fwd, recipe.py:27)
FP8_MAX_BWD = 57344.0   # e5m2


@dataclass
class DelayedScaling:
    margin: int = 0
    fp8_format: str = "HYBRID"
    amax_history_len: int = 1024
    amax_compute_algo: str = "max"
    scaling_factor_compute_algo: Optional[object] = None

    def __post_init__(self):
        if self.fp8_format != "HYBRID":
            raise ValueError("only Format.HYBRID is supported")
        if callable(self.amax_compute_algo) or self.scaling_factor_compute_algo is not None \
                or self.amax_compute_algo not in ("max", "most_recent"):
            raise ValueError("We only support the fp8 recipe with 'max' or 'most_recent' amax_compute_algo and default "
                             "scaling_factor_compute_algo at this moment.")


# ---- fp8_autocast (itex/python/fp8/autocast.py:26-68,122-151): a process-wide "FP8 on" flag and recipe that layers
# consult when they are built and called; nesting restores the outer state on exit.
_FP8_ENABLED = False
_FP8_RECIPE = None


def get_default_fp8_recipe():
    """Margin 0, HYBRID format, 'max' over the default history (autocast.py:42-47)."""
    return DelayedScaling()


def get_fp8_dtype(fp8_recipe, fwd=True):
    """HYBRID: e4m3 forward, e5m2 backward (autocast.py:49-52)."""
    assert fp8_recipe.fp8_format == "HYBRID"
    return "E4M3" if fwd else "E5M2"


def is_fp8_enabled():
    return _FP8_ENABLED


def get_fp8_recipe():
    return _FP8_RECIPE


@contextmanager
def fp8_autocast(enabled: bool = False, fp8_recipe: Optional[DelayedScaling] = None):
    """with fp8_autocast(enabled=True, fp8_recipe=DelayedScaling(...)): y = layer(x)"""
    global _FP8_ENABLED, _FP8_RECIPE
    saved = (_FP8_ENABLED, _FP8_RECIPE)
    try:
        _FP8_ENABLED = enabled
        _FP8_RECIPE = get_default_fp8_recipe() if fp8_recipe is None else fp8_recipe
        yield
    finally:
        _FP8_ENABLED, _FP8_RECIPE = saved


class Fp8Meta:
    """amax_history [H, n], scale [n], scale_inv [n] on one device (n = 3 * num_gemms forward)."""

    def __init__(self, recipe: DelayedScaling, num_gemms: int = 1, device="cuda", fwd: bool = True):
        n = num_gemms * (3 if fwd else 2)
        self.recipe = recipe
        self.fp8_max = FP8_MAX_FWD if fwd else FP8_MAX_BWD
        self.scale = torch.ones(n, dtype=torch.float32, device=device)
        self.scale_inv = torch.ones(n, dtype=torch.float32, device=device)
        self.amax_history = torch.zeros((recipe.amax_history_len, n), dtype=torch.float32, device=device)

    def amax_and_scale_update(self):
        """Run before the forward of each step (base.py:197-200)."""
        K.fp8_amax_and_scale_update(self.amax_history, self.scale, self.scale_inv, self.fp8_max,
                                    float(self.recipe.margin), self.recipe.amax_compute_algo)

    def save_blob(self) -> bytes:
        """The state as one host blob (itexb_fp8_meta_save): what a checkpoint stores for this layer."""
        import ctypes as C
        from . import _lib as L
        lib = L.load()
        lib.itexb_fp8_meta_blob_bytes.restype = C.c_size_t
        h, n = self.amax_history.shape
        nbytes = lib.itexb_fp8_meta_blob_bytes(h, n)
        buf = C.create_string_buffer(nbytes)
        L.check(lib.itexb_fp8_meta_save(C.c_void_p(self.amax_history.data_ptr()), C.c_void_p(self.scale.data_ptr()), C.c_void_p(self.scale_inv.data_ptr()),
                                        h, n, buf, C.c_size_t(nbytes), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return bytes(buf.raw)

    def load_blob(self, blob: bytes):
        import ctypes as C
        from . import _lib as L
        h, n = self.amax_history.shape
        L.check(L.load().itexb_fp8_meta_load(C.c_void_p(self.amax_history.data_ptr()), C.c_void_p(self.scale.data_ptr()),
                                             C.c_void_p(self.scale_inv.data_ptr()), h, n, blob, C.c_size_t(len(blob)),
                                             C.c_void_p(torch.cuda.current_stream().cuda_stream)))

    def state_dict(self):
        return {"scale": self.scale.clone(), "scale_inv": self.scale_inv.clone(), "amax_history": self.amax_history.clone()}

    def load_state_dict(self, sd):
        self.scale.copy_(sd["scale"])
        self.scale_inv.copy_(sd["scale_inv"])
        self.amax_history.copy_(sd["amax_history"])


class _DeviceBlock:
    """A raw device allocation seen by torch through the CUDA array interface (bytes)."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 2}


def peer_gather_layout(world, shard_bytes):
    """Byte layout of one rank's gather block.  shard_bytes: bytes of one rank's output shard for each linear served.
    Per linear, `world` slots of that many bytes (slot r receives rank r's shard; sizes must be multiples of 256 so every
    slot starts on the allocator's alignment), then two int32 flag rows of `world` entries - row "data": rank r's shards
    of the current step have arrived here; row "ack": rank r has finished reading the previous step's data - then the
    step counter and a status word.  Returns a dict of offsets; the same on every rank, so a peer's address of anything
    is that peer's base plus the local offset."""
    offs, off = [], 0
    for b in shard_bytes:
        if b <= 0 or b % 256 != 0:
            raise ValueError("shard sizes must be positive multiples of 256 bytes, got %d" % b)
        offs.append(off)
        off += b * world
    lay = {"linear": offs, "data_flags": off, "ack_flags": off + 4 * world, "counter": off + 8 * world, "status": off + 8 * world + 4}
    lay["total"] = (off + 8 * world + 8 + 255) // 256 * 256
    return lay


def peer_slot_offset(layout, shard_bytes, linear, src_rank):
    """Offset (in every rank's block) of the slot that holds `src_rank`'s shard of linear `linear`."""
    return layout["linear"][linear] + shard_bytes[linear] * src_rank


class PeerGather:
    """All-gather of column-parallel outputs by peer stores: every rank owns a [world, M, N/world] buffer in memory that all
    ranks of the node have mapped (CUDA IPC); rank r's GEMM kernel copies its shard, tile by tile, into slot r of EVERY rank's buffer
    while it is being computed (itexb_gemm with peer_out), so no separate collective runs afterwards.

    Protocol per step, all on the caller's stream (values are a device-side step counter, so a captured step replays):
      begin()    counter += 1; wait until every peer has acknowledged consuming the previous step (nobody overwrites a
                 buffer that is still being read);
      ...GEMMs with out=local(i) and peer_out=peers(i) ...
      publish()  make the stores visible, tell every rank "my shard of this step is in your buffer";
      finish()   wait (bounded: a missing peer becomes a status, not a hang) until all shards have arrived here; the
                 gathered buffers may be read from here on; acknowledge() after the last read.
    One PeerGather serves several linears: give their shard sizes as `shard_shapes`."""

    def __init__(self, shard_shapes, dtype, rank, world, device, exchange):
        """exchange(obj) -> list of every rank's obj (e.g. torch.distributed.all_gather_object wrapped); host plumbing only."""
        import ctypes as C
        from . import _lib as L
        assert 2 <= world <= 8, "PeerGather serves the GPUs of one node"
        self.lib, self.L, self.C = L.load(), L, C
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.ordinal = self.device.index or 0
        esz = torch.empty(0, dtype=dtype).element_size()
        self.shapes = [tuple(sh) for sh in shard_shapes]
        self.shard_bytes = [m * n * esz for (m, n) in self.shapes]
        self.layout = peer_gather_layout(world, self.shard_bytes)
        self.data_flags_off, self.ack_flags_off = self.layout["data_flags"], self.layout["ack_flags"]
        self.counter_off, self.status_off, self.nbytes = self.layout["counter"], self.layout["status"], self.layout["total"]
        base = C.c_void_p()
        L.check(self.lib.itexb_rt_allocate(self.ordinal, self.nbytes, C.byref(base)))
        self.base = base.value
        self.block = torch.as_tensor(_DeviceBlock(self.base, self.nbytes), device=self.device)
        self.block.zero_()
        torch.cuda.synchronize(self.device)
        handle = C.create_string_buffer(64)
        L.check(self.lib.itexb_rt_ipc_export(C.c_void_p(self.base), handle))
        handles = exchange(bytes(handle.raw))
        self.peer_base = {}
        for r, h in enumerate(handles):
            if r == rank:
                continue
            p = C.c_void_p()
            L.check(self.lib.itexb_rt_ipc_open(C.create_string_buffer(h, 64), C.byref(p)))
            self.peer_base[r] = p.value
        self.dtype = dtype
        all_bases = [self.base if r == rank else self.peer_base[r] for r in range(world)]
        self._data_flag_ptrs = (C.c_void_p * world)(*[b + self.data_flags_off + 4 * rank for b in all_bases])
        self._ack_flag_ptrs = (C.c_void_p * world)(*[b + self.ack_flags_off + 4 * rank for b in all_bases])
        exchange(0)   # every rank has opened every block before anyone stores into one

    def gathered(self, i):
        """[world, M, N/world] view of linear i's gather buffer on this rank."""
        off, (m, n) = self.layout["linear"][i], self.shapes[i]
        return self.block[off:off + self.shard_bytes[i] * self.world].view(self.dtype).view(self.world, m, n)

    def local(self, i):
        """This rank's own slot of linear i: the `out` of its GEMM."""
        return self.gathered(i)[self.rank]

    def peers(self, i):
        """Addresses of this rank's slot in every other rank's buffer of linear i: the `peer_out` of its GEMM."""
        off = peer_slot_offset(self.layout, self.shard_bytes, i, self.rank)
        return [self.peer_base[r] + off for r in range(self.world) if r != self.rank]

    @property
    def status(self):
        return self.block[self.status_off:self.status_off + 4].view(torch.int32)

    def _stream(self):
        return self.C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def begin(self):
        self.L.check(self.lib.itexb_peer_advance(self.C.c_void_p(self.base + self.counter_off), self._stream()))
        # acknowledgements carry the number of the step that was consumed: wait for (this step - 1)
        self.L.check(self.lib.itexb_peer_wait(self.C.c_void_p(self.base + self.ack_flags_off), self.world, -1,
                                              self.C.c_void_p(self.base + self.counter_off), self.C.c_void_p(self.base + self.status_off), self._stream()))

    def publish(self):
        self.L.check(self.lib.itexb_peer_signal(self._data_flag_ptrs, self.world, 0, self.C.c_void_p(self.base + self.counter_off), self._stream()))

    def finish(self):
        self.L.check(self.lib.itexb_peer_wait(self.C.c_void_p(self.base + self.data_flags_off), self.world, 0,
                                              self.C.c_void_p(self.base + self.counter_off), self.C.c_void_p(self.base + self.status_off), self._stream()))

    def acknowledge(self):
        self.L.check(self.lib.itexb_peer_signal(self._ack_flag_ptrs, self.world, 0, self.C.c_void_p(self.base + self.counter_off), self._stream()))

    def linears(self, layers, inputs, reduce_amax=None, streams=True):
        """One step of column-parallel Fp8Dense layers that do not depend on one another: begin(), layer i on inputs[i] with
        its product gathered into buffer i, publish(), finish().  Returns the gathered buffers; the caller reads them and then
        calls acknowledge().

        streams: every layer runs on a stream of its own (forked from and joined to the caller's), the widest shard launched
        first, so one layer's quantize passes and main loop run under another's copies and NVLink stays busy from the first
        finished tile to the last; otherwise all on the caller's stream, in order.
        reduce_amax(rows): the caller's collective over the layers' newest amax rows (max over the ranks, in place; e.g. one
        coalesced NCCL all-reduce), so that every rank keeps the same scaling state.  It runs on a side stream and is joined
        before return; with `streams` it is launched between the quantize passes and the GEMMs (a collective kernel launched
        later finds no free SM while persistent GEMMs hold all of them, and its whole latency lands at the end of the step).
        Captures into a CUDA graph like any fork/join of streams."""
        assert len(layers) == len(inputs) == len(self.shapes)
        main = torch.cuda.current_stream(self.device)
        if streams and getattr(self, "_lanes", None) is None:
            self._lanes = [torch.cuda.Stream(device=self.device) for _ in layers]
        if reduce_amax is not None and getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(device=self.device, priority=-1)
        rows = [layer.meta.amax_history[0] for layer in layers]
        self.begin()
        if streams:
            order = sorted(range(len(layers)), key=lambda i: -self.shapes[i][1])
            quantized = {}
            for i in order:
                self._lanes[i].wait_stream(main)
                with torch.cuda.stream(self._lanes[i]):
                    quantized[i] = layers[i].quantize_inputs(inputs[i])
                if reduce_amax is not None:
                    self._side.wait_stream(self._lanes[i])
            if reduce_amax is not None:
                # the rows are final once the quantize passes are done: the collective is launched before the GEMMs take
                # the SMs and runs under them
                with torch.cuda.stream(self._side):
                    reduce_amax(rows)
            for i in order:
                with torch.cuda.stream(self._lanes[i]):
                    layers[i].gathered_matmul(*quantized[i], self, i)
            for lane in self._lanes:
                main.wait_stream(lane)
        else:
            for i, layer in enumerate(layers):
                layer(inputs[i], gather=self, gather_index=i)
            if reduce_amax is not None:
                self._side.wait_stream(main)
                with torch.cuda.stream(self._side):
                    reduce_amax(rows)
        self.publish()
        self.finish()
        if reduce_amax is not None:
            main.wait_stream(self._side)
        return [self.gathered(i) for i in range(len(layers))]

    def close(self, barrier=None):
        """Unmaps the peers' blocks and frees this rank's; `barrier()` (a host rendezvous) makes sure no rank frees its
        block while another still has kernels in flight that store into it."""
        torch.cuda.synchronize(self.device)
        if barrier is not None:
            barrier()
        for p in self.peer_base.values():
            self.lib.itexb_rt_ipc_close(self.C.c_void_p(p))
        self.peer_base = {}
        if barrier is not None:
            barrier()
        if self.base:
            self.block = None
            self.lib.itexb_rt_deallocate(self.ordinal, self.C.c_void_p(self.base))
            self.base = 0


class Fp8Dense:
    """Forward of the FP8 Dense layer: y = x @ kernel (+ bias), e4m3 operands, `out_dtype` result.

    kernel is [in, out] like the Keras layer's weight; with `weight_layout="nk"` the caller
    keeps it as [out, in] and the op runs with transpose_b=True (no per-call transposition).
    """

    def __init__(self, kernel: torch.Tensor, bias: Optional[torch.Tensor] = None, recipe: Optional[DelayedScaling] = None,
                 out_dtype="bfloat16", weight_layout="kn"):
        self.kernel = kernel
        self.bias = bias
        self.recipe = recipe or (get_fp8_recipe() if is_fp8_enabled() else None) or DelayedScaling()  # explicit, autocast's, default
        self.meta = Fp8Meta(self.recipe, 1, kernel.device, fwd=True)
        self.out_dtype = out_dtype
        self.transpose_b = weight_layout == "nk"
        self._dummy = torch.zeros(1, dtype=torch.bfloat16 if out_dtype == "bfloat16" else torch.float32, device=kernel.device)
        self._nodes = {}    # the layer's kernel instances, one per node of its graph, kept across calls

    def _quantize(self, t: torch.Tensor, index: int) -> torch.Tensor:
        key = ("q", index, t.dtype)
        if key not in self._nodes:
            self._nodes[key] = ops.Op("Fp8Quantize", in_dtype=ops._TORCH_TO_DT[t.dtype], fp8_meta_index=index, fp8_dtype="E4M3")
        return self._nodes[key](t, self.meta.amax_history[0], self.meta.scale)

    def _matmul(self, xq, wq, bias, out=None):
        from . import _lib as L
        if "mm" not in self._nodes:
            self._nodes["mm"] = ops.Op("Fp8Matmul", fp8_meta_index_a=0, fp8_meta_index_b=1, fp8_meta_index_c=-1, transpose_a=False,
                                       transpose_b=self.transpose_b, use_bias=self.bias is not None, has_post_add=False,
                                       sum_dtype=self.out_dtype, out_dtype=self.out_dtype, fp8_dtype_a="E4M3", fp8_dtype_b="E4M3",
                                       fp8_dtype_c="")
        m = self.meta
        return self._nodes["mm"](xq, wq, bias, self._dummy, m.scale_inv, m.scale_inv, m.amax_history[0], m.scale,
                                 dtypes={0: L.DT_INT8, 1: L.DT_INT8}, out=None if out is None else {0: out})

    def quantize_inputs(self, x: torch.Tensor, update_meta: bool = True):
        """First half of the forward: the scale update and the two Fp8Quantize passes.  Returns (xq, wq); after it the newest
        amax row holds this call's maxima (a bf16 / f32 product adds none)."""
        if update_meta:
            self.meta.amax_and_scale_update()
        return self._quantize(x, 0), self._quantize(self.kernel, 1)

    def gathered_matmul(self, xq, wq, gather, gather_index: int = 0) -> torch.Tensor:
        """Second half for a column-parallel layer (kernel kept as [N/world, K]): the product lands in slot `rank` of linear
        `gather_index`'s buffer on every rank of the PeerGather, stored by the GEMM kernel's copying warps; returns this
        rank's slot.  The arithmetic is that of the Fp8Matmul op (same kernel, same scales)."""
        from . import _lib as L
        assert self.transpose_b and self.bias is None and self.out_dtype == "bfloat16", "the fused gather path serves [N,K] kernels, bf16 out"
        m = self.meta
        ep = K.make_epilogue(alpha_a=m.scale_inv[0:1], alpha_b=m.scale_inv[1:2])
        out = gather.local(gather_index)
        K.gemm(xq.view(torch.uint8), wq.view(torch.uint8), L.DT_BFLOAT16, a_dtype=L.DT_FP8_E4M3, b_dtype=L.DT_FP8_E4M3, ep=ep, out=out,
               peer_out=gather.peers(gather_index), status_word=gather.status)
        return out

    def __call__(self, x: torch.Tensor, update_meta: bool = True, gather=None, gather_index: int = 0, out=None) -> torch.Tensor:
        """gather: a PeerGather; see gathered_matmul."""
        xq, wq = self.quantize_inputs(x, update_meta)
        if gather is not None:
            return self.gathered_matmul(xq, wq, gather, gather_index)
        bias = self.bias if self.bias is not None else self._dummy
        return self._matmul(xq, wq, bias, out)      # out: the product is written into the caller's [M, N] tensor
