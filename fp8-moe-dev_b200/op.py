"""Host-side mirror of the reference operator.

`run(...)` takes the same eleven positional arguments, in the same order and with the same
dtypes and layouts, as the reference's `run` (kernel/moe_fp8.cu:2663-2669), writes the bf16
result into `output` (destination passing) and returns without synchronising.  `MoeLayer`
is the explicit-handle form of the same call.  Torch is used only for device memory and
the current stream; all compute happens in libmoe_fp8_b200.so.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import numpy as np
import torch

from . import _lib

H, I, N1, NE = 7168, 2048, 4096, 256


class MoeError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"moe_fp8_b200 error {code}: {message}")
        self.code = code


def _check_tensor(name, t, dtype, shape, device=None):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if device is not None and t.device != device:
        raise ValueError(f"{name} must live on {device}, got {t.device}")


class _DeviceSpan:
    """A borrowed range of device memory, presented through the CUDA array interface."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = dict(shape=tuple(shape), typestr=typestr, data=(int(ptr), False), version=3,
                                             strides=None)


def _device_view(ptr, shape, typestr, device):
    """torch tensor over memory the library owns (no copy)."""
    return torch.as_tensor(_DeviceSpan(ptr, shape, typestr), device=torch.device("cuda", device))


class MoeLayer:
    """One handle = one GPU's workspace for up to `max_tokens` tokens and `num_local_experts`
    experts (32 per reference shard; 64/128/256 hold several shards on one GPU)."""

    def __init__(self, max_tokens: int, num_local_experts: int = 32, device: Optional[int] = None, *,
                 hidden: int = H, intermediate: int = I, top_k: int = 8, n_group: int = 8, topk_group: int = 4):
        """The keyword arguments select another shape of the layer (hidden a multiple of 256, intermediate of
        128, both at most 8192; top_k <= 8; n_group 1, 2, 4 or 8); the defaults are the reference's."""
        self._lib = _lib.load()
        if device is None:
            device = torch.cuda.current_device()
        self.device = int(device)
        self.max_tokens = int(max_tokens)
        self.num_local_experts = int(num_local_experts)
        self.hidden, self.intermediate = int(hidden), int(intermediate)
        self.top_k, self.n_group, self.topk_group = int(top_k), int(n_group), int(topk_group)
        shape = _lib.Shape(self.hidden, self.intermediate, self.top_k, self.n_group, self.topk_group)
        h = C.c_void_p()
        rc = self._lib.moe_fp8_b200_create_shaped(C.byref(h), self.device, self.max_tokens, self.num_local_experts,
                                                  C.byref(shape))
        if rc != _lib.OK:
            raise MoeError(rc, self._lib.moe_fp8_b200_last_error(None).decode())
        self._h = h
        self.row_capacity = self._lib.moe_fp8_b200_row_capacity(self.max_tokens, self.num_local_experts)

    # -- lifetime ---------------------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None):
            self._lib.moe_fp8_b200_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _raise(self, rc):
        raise MoeError(rc, self._lib.moe_fp8_b200_last_error(self._h).decode())

    # -- options ----------------------------------------------------------------------
    def set_reference_pruning(self, on: bool):
        rc = self._lib.moe_fp8_b200_set_option(self._h, _lib.OPT_REFERENCE_PRUNING, int(bool(on)))
        if rc != _lib.OK:
            self._raise(rc)

    def set_exact_silu(self, on: bool):
        rc = self._lib.moe_fp8_b200_set_option(self._h, _lib.OPT_EXACT_SILU, int(bool(on)))
        if rc != _lib.OK:
            self._raise(rc)

    def set_decode_kernel(self, on: bool):
        """Batches of at most 8 tokens: one cooperative kernel (default) or the staged chain."""
        rc = self._lib.moe_fp8_b200_set_option(self._h, _lib.OPT_DECODE_KERNEL, int(bool(on)))
        if rc != _lib.OK:
            self._raise(rc)

    def set_stop_after_stage(self, stages: int):
        """Diagnostics: enqueue only the first `stages` stages of the chain (1 = routing, dispatch and the
        offset scan; 2 = + permute; 3 = + GEMM1; 4 = + GEMM2; 0 = everything)."""
        rc = self._lib.moe_fp8_b200_set_option(self._h, _lib.OPT_STOP_AFTER_STAGE, int(stages))
        if rc != _lib.OK:
            self._raise(rc)

    def set_wait_limit_us(self, us: int):
        """Bound of the fused reduce-scatter's wait for peer rows (default 1 s)."""
        rc = self._lib.moe_fp8_b200_set_option(self._h, _lib.OPT_WAIT_LIMIT_US, int(us))
        if rc != _lib.OK:
            self._raise(rc)

    def set_weight_prelayout(self, on: bool):
        """Tile-ordered copies of the weights for the chain's GEMMs (one contiguous 32 KB piece per tile and K
        block): allocates num_local_experts x the size of one expert's weights on the handle's device, filled
        once per weight pointer.  Same results; for batches that are bound by streaming the weights."""
        rc = self._lib.moe_fp8_b200_set_option(self._h, _lib.OPT_WEIGHT_PRELAYOUT, int(bool(on)))
        if rc != _lib.OK:
            self._raise(rc)

    def set_small_batch_ring(self, on: bool):
        """Batches of 5 to 64 tokens: 64-row activation boxes and a fourth operand stage in the GEMMs (default on)."""
        rc = self._lib.moe_fp8_b200_set_option(self._h, _lib.OPT_SMALL_BATCH_RING, int(bool(on)))
        if rc != _lib.OK:
            self._raise(rc)

    def inject_device_status(self, status: int, stale_barrier_arrivals: int = 0):
        """Host-side failure injection for tests of the error path (see the header)."""
        stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self._lib.moe_fp8_b200_inject_device_status(self._h, int(status), int(stale_barrier_arrivals),
                                                         C.c_void_p(stream))
        if rc != _lib.OK:
            self._raise(rc)

    def invalidate_weights(self):
        """Call after the weight-scale tensors' contents changed under the same addresses."""
        rc = self._lib.moe_fp8_b200_invalidate_weights(self._h)
        if rc != _lib.OK:
            self._raise(rc)

    def set_expert_stride(self, stride: int):
        """Strided expert placement (multi-GPU wrapper): this handle's experts are the global ids g
        with g % stride == local_expert_offset, stacked in increasing g; stride 1 = contiguous."""
        rc = self._lib.moe_fp8_b200_set_option(self._h, _lib.OPT_EXPERT_STRIDE, int(stride))
        if rc != _lib.OK:
            self._raise(rc)

    def set_expert_map(self, expert_ids):
        """Table placement: this handle's weight tensors hold the global experts `expert_ids`, in that
        order (None: back to the contiguous block at local_expert_offset)."""
        if expert_ids is None:
            rc = self._lib.moe_fp8_b200_set_expert_map(self._h, None)
        else:
            table = (C.c_int32 * NE)(*([-1] * NE))
            for slot, g in enumerate(expert_ids):
                table[int(g)] = slot
            rc = self._lib.moe_fp8_b200_set_expert_map(self._h, table)
        if rc != _lib.OK:
            self._raise(rc)

    STAGES = ("route_dispatch", "scan", "permute", "gemm1", "gemm2", "combine")

    def set_stage_timing(self, on: bool):
        rc = self._lib.moe_fp8_b200_set_option(self._h, _lib.OPT_STAGE_TIMING, int(bool(on)))
        if rc != _lib.OK:
            self._raise(rc)

    def stage_times(self):
        """({stage: mean ms}, runs) over the runs since stage timing was switched on."""
        ms = (C.c_float * 6)()
        n = C.c_int(0)
        rc = self._lib.moe_fp8_b200_stage_times(self._h, ms, C.byref(n))
        if rc != _lib.OK:
            self._raise(rc)
        return dict(zip(self.STAGES, [float(x) for x in ms])), int(n.value)

    # -- the operator -----------------------------------------------------------------
    def _args(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
              gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
              routed_scaling_factor, output, host: bool, out_rows: Optional[int] = None):
        T = int(routing_logits.shape[0])
        E = self.num_local_experts
        dev = torch.device("cuda", self.device)
        io_dev = torch.device("cpu") if host else dev
        _check_tensor("routing_logits", routing_logits, torch.float32, (T, NE), io_dev)
        _check_tensor("routing_bias", routing_bias, torch.bfloat16, (NE,), dev)
        H, I = self.hidden, self.intermediate
        N1 = 2 * I
        _check_tensor("hidden_states", hidden_states, torch.float8_e4m3fn, (T, H), io_dev)
        _check_tensor("hidden_states_scale", hidden_states_scale, torch.float32, (H // 128, T), io_dev)
        _check_tensor("gemm1_weights", gemm1_weights, torch.float8_e4m3fn, (E, N1, H), dev)
        _check_tensor("gemm1_weights_scale", gemm1_weights_scale, torch.float32, (E, N1 // 128, H // 128), dev)
        _check_tensor("gemm2_weights", gemm2_weights, torch.float8_e4m3fn, (E, H, I), dev)
        _check_tensor("gemm2_weights_scale", gemm2_weights_scale, torch.float32, (E, H // 128, I // 128), dev)
        if output is not None:
            _check_tensor("output", output, torch.bfloat16, (T if out_rows is None else out_rows, H), io_dev)
        a = _lib.Args()
        a.routing_logits = routing_logits.data_ptr()
        a.routing_bias = routing_bias.data_ptr()
        a.hidden_states = hidden_states.data_ptr()
        a.hidden_states_scale = hidden_states_scale.data_ptr()
        a.gemm1_weights = gemm1_weights.data_ptr()
        a.gemm1_weights_scale = gemm1_weights_scale.data_ptr()
        a.gemm2_weights = gemm2_weights.data_ptr()
        a.gemm2_weights_scale = gemm2_weights_scale.data_ptr()
        a.local_expert_offset = int(local_expert_offset)
        a.routed_scaling_factor = float(routed_scaling_factor)
        a.output = output.data_ptr() if output is not None else None
        a.num_tokens = T
        return a

    def run(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
            gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset, routed_scaling_factor,
            output, stream: Optional[int] = None):
        """Device tensors in, bf16 `output` overwritten; asynchronous on the current stream."""
        a = self._args(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                       gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                       routed_scaling_factor, output, host=False)
        if stream is None:
            stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self._lib.moe_fp8_b200_run(self._h, C.byref(a), C.c_void_p(stream))
        if rc != _lib.OK:
            self._raise(rc)
        return output

    def run_reduce_scatter(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                           gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                           routed_scaling_factor, owned_output, peer_buffers, buffer_bytes: int, rank: int,
                           world: int, epoch: int, stream: Optional[int] = None, capacity_tokens: int = 0):
        """Expert-parallel run with the cross-rank sum fused into the combine step:
        `owned_output` [ceil(T / world), 7168] receives this rank's token slice of the summed
        output.  `peer_buffers` are the ranks' receive buffers as mapped into this process."""
        T = int(routing_logits.shape[0])
        per = (T + world - 1) // world
        a = self._args(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                       gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                       routed_scaling_factor, owned_output, host=False, out_rows=per)
        x = _lib.Exchange()
        for i, ptr in enumerate(peer_buffers):
            x.peer_buffers[i] = int(ptr)
        x.buffer_bytes, x.rank, x.world, x.epoch = int(buffer_bytes), int(rank), int(world), int(epoch) & 0xFFFFFFFF
        x.capacity_tokens = int(capacity_tokens)
        if stream is None:
            stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self._lib.moe_fp8_b200_run_reduce_scatter(self._h, C.byref(a), C.byref(x), C.c_void_p(stream))
        if rc != _lib.OK:
            self._raise(rc)
        return owned_output

    # -- the operators either side of the layer ----------------------------------------
    def quantize_hidden(self, x, q_out=None, scale_out=None, stream: Optional[int] = None):
        """bf16 x [T, 7168] (device) -> (e4m3 [T, 7168], fp32 scales [56, T]): the pair `run` takes."""
        T = int(x.shape[0])
        H = self.hidden
        dev = torch.device("cuda", self.device)
        _check_tensor("x", x, torch.bfloat16, (T, H), dev)
        if q_out is None:
            q_out = torch.empty((T, H), dtype=torch.float8_e4m3fn, device=dev)
        if scale_out is None:
            scale_out = torch.empty((H // 128, T), dtype=torch.float32, device=dev)
        _check_tensor("q_out", q_out, torch.float8_e4m3fn, (T, H), dev)
        _check_tensor("scale_out", scale_out, torch.float32, (H // 128, T), dev)
        if stream is None:
            stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self._lib.moe_fp8_b200_quantize_hidden(self._h, x.data_ptr(), T, q_out.data_ptr(), scale_out.data_ptr(),
                                                    C.c_void_p(stream))
        if rc != _lib.OK:
            self._raise(rc)
        return q_out, scale_out

    def run_unfinalized(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                        gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                        routed_scaling_factor, stream: Optional[int] = None):
        """The layer without the weighted combine.  Returns views INTO the workspace (valid until
        the next run on this layer): y bf16 [row_capacity, 7168], expert_offset int32 [E+1],
        pair_count int32 [T], pair_code int32 [T, 8] ((local expert << 24) | slot), pair_weight
        fp32 [T, 8]."""
        T = int(routing_logits.shape[0])
        a = self._args(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                       gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                       routed_scaling_factor, None, host=False)
        v = _lib.Unfinalized()
        if stream is None:
            stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self._lib.moe_fp8_b200_run_unfinalized(self._h, C.byref(a), C.byref(v), C.c_void_p(stream))
        if rc != _lib.OK:
            self._raise(rc)
        E, cap = self.num_local_experts, int(v.row_capacity)
        return dict(
            y=_device_view(v.y, (cap, self.hidden), "<i2", self.device).view(torch.bfloat16),
            expert_offset=_device_view(v.expert_offset, (E + 1,), "<i4", self.device),
            pair_count=_device_view(v.pair_count, (T,), "<i4", self.device),
            pair_code=_device_view(v.pair_code, (T, 8), "<i4", self.device),
            pair_weight=_device_view(v.pair_weight, (T, 8), "<f4", self.device))

    def finalize(self, num_tokens: int, output, stream: Optional[int] = None):
        """The weighted combine of the latest unfinalized run into bf16 `output` [T, 7168]."""
        _check_tensor("output", output, torch.bfloat16, (int(num_tokens), self.hidden), torch.device("cuda", self.device))
        if stream is None:
            stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self._lib.moe_fp8_b200_finalize(self._h, int(num_tokens), output.data_ptr(), C.c_void_p(stream))
        if rc != _lib.OK:
            self._raise(rc)
        return output

    def run_host(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                 gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                 routed_scaling_factor, output, stream: Optional[int] = None):
        """Per-call tensors (logits, hidden, hidden scale, output) in HOST memory; the call
        copies in, runs, copies out and synchronises."""
        a = self._args(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                       gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                       routed_scaling_factor, output, host=True)
        if stream is None:
            stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self._lib.moe_fp8_b200_run_host(self._h, C.byref(a), C.c_void_p(stream))
        if rc != _lib.OK:
            self._raise(rc)
        return output

    def run_host_async(self, routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                       gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                       routed_scaling_factor, output, stream: Optional[int] = None) -> int:
        """Pipelined run_host: enqueues copy-in, layer and copy-out and returns a ticket at once.
        The host tensors must stay untouched until host_wait(ticket); at most two calls in flight."""
        a = self._args(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                       gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, local_expert_offset,
                       routed_scaling_factor, output, host=True)
        if stream is None:
            stream = torch.cuda.current_stream(self.device).cuda_stream
        ticket = C.c_int64(-1)
        rc = self._lib.moe_fp8_b200_run_host_async(self._h, C.byref(a), C.c_void_p(stream), C.byref(ticket))
        if rc != _lib.OK:
            self._raise(rc)
        return int(ticket.value)

    def host_wait(self, ticket: int):
        rc = self._lib.moe_fp8_b200_host_wait(self._h, int(ticket))
        if rc != _lib.OK:
            self._raise(rc)

    def check(self, stream: Optional[int] = None):
        """Synchronise and raise if a kernel recorded a failure (e.g. a wait that ran out)."""
        if stream is None:
            stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self._lib.moe_fp8_b200_check(self._h, C.c_void_p(stream))
        if rc != _lib.OK:
            self._raise(rc)

    # -- diagnostics ------------------------------------------------------------------
    _DTYPES = dict(expert_count=np.int32, expert_offset=np.int32, topk_idx=np.int32, topk_weight=np.float32,
                   pair_count=np.int32, pair_code=np.uint32, pair_weight=np.float32, num_tiles=np.int32,
                   row_token=np.int32, a1=np.uint8, sfa1=np.float32, a2=np.uint8, sfa2=np.float32, y=np.uint16,
                   status=np.int32, decode_timeline=np.uint64, exchange_timeline=np.uint64, pair_row=np.int32)

    def read(self, name: str, count: int, offset_elems: int = 0) -> np.ndarray:
        """First `count` elements (after `offset_elems`) of an intermediate buffer of the last run."""
        dt = np.dtype(self._DTYPES[name])
        out = np.empty(int(count), dtype=dt)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self._lib.moe_fp8_b200_read_intermediate(
            self._h, _lib.BUF[name], out.ctypes.data_as(C.c_void_p), out.nbytes, int(offset_elems) * dt.itemsize,
            C.c_void_p(stream))
        if rc != _lib.OK:
            self._raise(rc)
        return out


# ----------------------------------------------------------------------------------------
# The reference-shaped entry point: one grow-only handle per (device, expert count), like
# the reference's thread-local workspace (kernel/moe_fp8.cu:2677-2689).
def expert_loads(routing_logits, routing_bias, routed_scaling_factor: float = 1.0, reference_pruning: bool = True):
    """Routed rows per global expert (256 counts, a CPU list) for the first <= 4096 tokens of a
    batch: the calibration input of the load-aware expert placement.  Runs the library's routing
    kernel alone (no weights needed).  The dispatch policy is keyed on the batch size, so the
    counts are those of a batch of min(T, 4096) tokens: for a longer batch they are taken under the
    4096-token policy (keep at most 3 per shard and renormalise, no drop-third rule), which slightly
    over-counts the rows of a T >= 10000 run but ranks the experts the same way."""
    T = min(int(routing_logits.shape[0]), _lib.NOALLOC_MAX_TOKENS)
    lg = routing_logits[:T].contiguous()
    dev = lg.device
    with torch.cuda.device(dev):   # the entry point works on the current device
        idx = torch.empty((max(T, 1), 8), dtype=torch.int32, device=dev)
        w = torch.empty((max(T, 1), 8), dtype=torch.float32, device=dev)
        cnt = torch.zeros((NE,), dtype=torch.int32, device=dev)
        err = C.create_string_buffer(256)
        stream = torch.cuda.current_stream(dev).cuda_stream
        rc = _lib.load().moe_fp8_b200_route_noalloc(lg.data_ptr(), routing_bias.data_ptr(), T, 0, NE,
                                                    float(routed_scaling_factor), int(reference_pruning), idx.data_ptr(),
                                                    w.data_ptr(), cnt.data_ptr(), C.c_void_p(stream), err, len(err))
        if rc != _lib.OK:
            raise MoeError(rc, err.value.decode())
        return [int(x) for x in cnt.cpu().tolist()]


_layers: Dict[Tuple[int, int], MoeLayer] = {}


def run(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
        gemm2_weights, gemm2_weights_scale, local_expert_offset, routed_scaling_factor, output):
    """Drop-in for the reference's `run` (destination passing, returns None)."""
    T = int(routing_logits.shape[0])
    if T <= 0:
        return None
    dev = routing_logits.device.index if routing_logits.is_cuda else torch.cuda.current_device()
    E = int(gemm1_weights.shape[0])
    key = (dev, E)
    layer = _layers.get(key)
    if layer is None or layer.max_tokens < T:
        if layer is not None:
            layer.close()
        layer = MoeLayer(max(T, 16), E, dev)
        _layers[key] = layer
    layer.run(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
              gemm2_weights, gemm2_weights_scale, local_expert_offset, routed_scaling_factor, output)
    return None
