"""``CUDAFusedInference``: the reference's fused decode engine
(cuda_fused_infer.go:75-459, cuda_fused_infer_q4.go:46-266) as a thin Python
class over the ``mg_*`` C ABI.  Method names and argument meaning follow the
Go type; all arithmetic runs in libmongoose_kernels.so on the GPU.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .configs import ModelConfig


class MongooseError(RuntimeError):
    pass


class GraphCaptureConfig:
    """GraphCaptureConfig (cuda_graph.go:293-298).  StreamCount and PipelineBreak are accepted for
    source compatibility; the engine runs a layer range on one stream."""

    def __init__(self, LayerStart: int = 0, LayerEnd: int = 0, StreamCount: int = 1, PipelineBreak: int = 0):
        self.LayerStart, self.LayerEnd = LayerStart, LayerEnd
        self.StreamCount, self.PipelineBreak = StreamCount, PipelineBreak


class CUDAGraph:
    """CUDAGraph (cuda_graph.go:300-311): a replayable layer range.  The engine keeps its own cached
    graphs (or the persistent kernel) and reads the position from device memory, so the handle only
    remembers the range."""

    def __init__(self, engine: "CUDAFusedInference", cfg: GraphCaptureConfig):
        self._eng, self.config, self.captured = engine, cfg, True

    def Launch(self, pos: int) -> None:
        """Replay at `pos` on the device-resident hidden state; asynchronous (cuda_graph.go:663-671)."""
        if not self.captured:
            return
        e = self._eng
        e._check(e._lib.mg_graph_launch(e._h, pos, self.config.LayerStart, self.config.LayerEnd), "CUDAGraph.Launch")

    def Destroy(self) -> None:
        self.captured = False


def _np_ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class CUDAFusedInference:
    def __init__(self, cfg: ModelConfig, device: int = 0, tp_rank: int = 0, tp_size: int = 1,
                 tp_id: bytes | None = None):
        """NewCUDAFusedInference (cuda_fused_infer.go:144).  With tp_size > 1 this process is one
        rank of a tensor-parallel group: tp_id is the 128-byte communicator id rank 0 made
        (mongoose_b200.multi.tp_unique_id), the call is collective, and every rank then sets the
        full weights and keeps its part."""
        self.cfg = cfg
        self._lib = _lib.load()
        c = _lib.MgConfig(dim=cfg.dim, kv_dim=cfg.kv_dim, head_dim=cfg.head_dim, n_heads=cfg.n_heads,
                          n_kv_heads=cfg.n_kv_heads, ffn_dim=cfg.ffn_dim, vocab=cfg.vocab,
                          n_layers=cfg.n_layers, max_seq=cfg.max_seq, rope_theta=float(cfg.rope_theta),
                          rms_eps=float(cfg.eps), layer_fmt=cfg.layer_fmt, head_fmt=cfg.head_fmt,
                          device=device, max_batch=1, flags=0)
        h = C.c_void_p()
        rc = self._lib.mg_create(C.byref(c), C.byref(h))
        if rc != 0 or not h.value:
            raise MongooseError(f"mg_create failed with status {rc} (is a B200 visible as device {device}?)")
        self._h = h
        self.tp_rank, self.tp_size = tp_rank, tp_size
        if tp_size > 1:
            if tp_id is None or len(tp_id) < 128:
                raise MongooseError("tensor parallelism needs the 128-byte communicator id")
            buf = C.create_string_buffer(bytes(tp_id), len(tp_id))
            self._check(self._lib.mg_tp_init(self._h, tp_rank, tp_size, buf, len(tp_id)), "mg_tp_init")

    # -- lifetime ---------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None):
            self._lib.mg_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def _check(self, rc: int, what: str):
        if rc != 0:
            raise MongooseError(f"{what}: status {rc}: {self._lib.mg_last_error(self._h).decode()}")

    # -- weights ----------------------------------------------------------
    def NumWeights(self) -> int:
        return self._lib.mg_num_weights(self._h)

    def SetWeight(self, idx: int, data) -> None:
        """fp32 tensor for slot idx = layer*12 + w; matrices are quantized on the
        host to the slot's format (cuda_fused_infer.go:241-272)."""
        a = np.ascontiguousarray(data, dtype=np.float32)
        self._check(self._lib.mg_set_weight(self._h, idx, _np_ptr(a), a.size), f"SetWeight({idx})")

    def SetWeightRaw(self, idx: int, blocks, fmt: int) -> None:
        """Raw quantized blocks for a matrix slot (SetWeightQ4_0, cuda_fused_infer_q4.go:46-90)."""
        a = np.ascontiguousarray(blocks).view(np.uint8)
        self._check(self._lib.mg_set_weight_raw(self._h, idx, _np_ptr(a), a.size, fmt), f"SetWeightRaw({idx})")

    def SetWeightQ4_0(self, idx: int, blocks) -> None:
        from .configs import FMT_Q4_0
        self.SetWeightRaw(idx, blocks, FMT_Q4_0)

    def BuildFusedDispatch(self) -> None:
        self._check(self._lib.mg_build(self._h), "BuildFusedDispatch")

    def ResetKV(self) -> None:
        self._check(self._lib.mg_reset_kv(self._h), "ResetKV")

    # -- stepping ---------------------------------------------------------
    def PartialStep(self, hiddenIn, pos: int, layerStart: int, layerEnd: int, hiddenOut=None,
                    logitsOut=None) -> int:
        """hiddenIn/hiddenOut/logitsOut are host float32 arrays (numpy, or pinned torch CPU
        tensors); returns 0 like the reference (cuda_fused_infer.go:392-459)."""
        rc = self._lib.mg_partial_step(self._h, _host_ptr(hiddenIn), pos, layerStart, layerEnd,
                                       _host_ptr(hiddenOut), _host_ptr(logitsOut))
        self._check(rc, "PartialStep")
        return 0

    # -- fp16 weights (cuda_fused_infer.go:274-361, cuda_fused_infer_fp16.go:201-282) ------------
    @property
    def WeightsFP16(self) -> bool:
        from .configs import FMT_F16
        return self.cfg.layer_fmt == FMT_F16 and self.cfg.head_fmt == FMT_F16

    def _require_fp16(self, what: str):
        if not self.WeightsFP16:
            raise MongooseError(f"{what}: this engine was created for quantized weights; create it with "
                                f"layer_fmt = head_fmt = FMT_F16 (one format per engine)")

    def SetWeightFP16(self, idx: int, data) -> None:
        """fp32 tensor stored as fp16, no quantization; norms stay fp32 and biases are skipped, as
        in the reference (cuda_fused_infer.go:276-316)."""
        self._require_fp16("SetWeightFP16")
        if idx < self.cfg.n_layers * 12 and idx % 12 in (4, 5, 6):
            return
        self.SetWeight(idx, data)

    def SetWeightRawFP16(self, idx: int, fp16Bytes, nElems: int, normData=None) -> None:
        """Raw fp16 bytes for matrix slots, normData (fp32) for norm slots, biases skipped
        (cuda_fused_infer.go:318-361)."""
        from .configs import FMT_F16
        self._require_fp16("SetWeightRawFP16")
        nL = self.cfg.n_layers
        w = idx % 12 if idx < nL * 12 else -1
        if w in (4, 5, 6):
            return
        if w in (0, 8) or idx == nL * 12:
            self.SetWeight(idx, normData)
            return
        a = np.ascontiguousarray(fp16Bytes).view(np.uint8)
        if a.size != 2 * nElems:
            raise MongooseError(f"SetWeightRawFP16({idx}): {a.size} bytes for {nElems} elements")
        self.SetWeightRaw(idx, a, FMT_F16)

    def PartialStepFP16(self, hiddenIn, pos: int, layerStart: int, layerEnd: int, hiddenOut=None,
                        logitsOut=None) -> int:
        """PartialStep on fp16 weights (cuda_fused_infer_fp16.go:201-282): the same fused kernels
        with the fp16 weight path instead of M=1 cuBLAS calls."""
        self._require_fp16("PartialStepFP16")
        return self.PartialStep(hiddenIn, pos, layerStart, layerEnd, hiddenOut, logitsOut)

    # -- GGUF Q4_0 names (cuda_fused_infer_q4.go:92-444) ----------------------------------------
    # The engine's format is fixed at creation (layer_fmt / head_fmt), so the Q4_0 entry points are the
    # same calls on an engine created with Q4_0 layers; they refuse an engine of another format.
    def _require_q4(self, what: str):
        if self.cfg.layer_fmt != 1:
            raise MongooseError(f"{what}: this engine was not created with Q4_0 layers (layer_fmt {self.cfg.layer_fmt})")

    def PartialStepQ4(self, hiddenIn, pos: int, layerStart: int, layerEnd: int, hiddenOut=None, logitsOut=None) -> int:
        self._require_q4("PartialStepQ4")
        return self.PartialStep(hiddenIn, pos, layerStart, layerEnd, hiddenOut, logitsOut)

    def PartialStepQ4Continue(self, pos: int, layerStart: int, layerEnd: int, hiddenOut=None, logitsOut=None) -> int:
        self._require_q4("PartialStepQ4Continue")
        return self.PartialStepContinue(pos, layerStart, layerEnd, hiddenOut, logitsOut)

    def PartialStepQ4ContinueOnStream1(self, pos: int, layerStart: int, layerEnd: int, logitsOut=None) -> int:
        """Asynchronous (cuda_fused_infer_q4.go:391-444): read the results after SyncStream1()."""
        self._require_q4("PartialStepQ4ContinueOnStream1")
        return self.PartialStepContinueOnStream1(pos, layerStart, layerEnd, logitsOut)

    def PartialStepContinueOnStream1(self, pos: int, layerStart: int, layerEnd: int, logitsOut=None) -> int:
        self._check(self._lib.mg_partial_step_continue_on_stream1(self._h, pos, layerStart, layerEnd, _host_ptr(logitsOut)),
                    "PartialStepContinueOnStream1")
        return 0

    def StepLayerResident(self, layer: int, pos: int, hiddenIn=None, preOut=None, postOut=None, logitsOut=None) -> None:
        """One layer with snapshots of the hidden state before and after it (+ logits), the call the
        reference's needle trainers drive (cuda_fused_infer_q4.go:451-605)."""
        self._check(self._lib.mg_step_layer_resident(self._h, layer, pos, _host_ptr(hiddenIn), _host_ptr(preOut),
                                                     _host_ptr(postOut), _host_ptr(logitsOut)), "StepLayerResident")

    # -- vNodes (cuda_fused_infer.go:630-684) -----------------------------------------------------
    def SetVNodeCount(self, n: int) -> None:
        self._check(self._lib.mg_set_vnode_count(self._h, n), "SetVNodeCount")

    def VNodeCount(self) -> int:
        return int(self._lib.mg_vnode_count(self._h))

    def RecordStageDone(self) -> None:
        self._check(self._lib.mg_record_stage_done(self._h), "RecordStageDone")

    def WaitStageDone(self) -> None:
        self._check(self._lib.mg_wait_stage_done(self._h), "WaitStageDone")

    def SyncStream1(self) -> None:
        self._check(self._lib.mg_sync_stream1(self._h), "SyncStream1")

    def QueueHiddenToL3OnStream1(self) -> None:
        self._check(self._lib.mg_queue_hidden_to_l3_on_stream1(self._h), "QueueHiddenToL3OnStream1")

    def SwapHiddenBuffer(self) -> None:
        """The reference alternates two hidden buffers so that an upload cannot overtake the L3 copy
        (cuda_fused_infer.go:733-737); here the copy is ordered before the next step by an event, so
        there is nothing to swap."""

    def DisableFusedDispatch(self) -> None:
        """The reference can fall back from its one-call dispatch to 17 calls per layer
        (cuda_fused_infer.go:739-742); this engine has one path."""

    # -- layer-range pipeline (cuda_fused_infer.go:461-737) -------------------------------------
    def SetLayerRange(self, layerStart: int, layerEnd: int) -> None:
        """This engine is a pipeline stage holding layers [layerStart, layerEnd); the last stage also
        holds the final norm and lm_head (cuda_fused_infer.go:542-556)."""
        self._check(self._lib.mg_set_layer_range(self._h, layerStart, layerEnd), "SetLayerRange")

    def PartialStepContinue(self, pos: int, layerStart: int, layerEnd: int, hiddenOut=None, logitsOut=None) -> int:
        """PartialStep without the upload: the hidden state is already on the device
        (cuda_fused_infer.go:463-528)."""
        rc = self._lib.mg_partial_step_continue(self._h, pos, layerStart, layerEnd, _host_ptr(hiddenOut),
                                                _host_ptr(logitsOut))
        self._check(rc, "PartialStepContinue")
        return 0

    def QueueHiddenTo(self, nxt: "CUDAFusedInference") -> None:
        """Hand the device-resident hidden state to the next stage (peer copy over NVLink between
        GPUs); asynchronous.  Replaces the reference's hop through host memory."""
        self._check(self._lib.mg_queue_hidden_to(self._h, nxt._h), "QueueHiddenTo")

    def WaitMailbox(self, timeout_ms: int = 1000) -> None:
        """Returns once the hidden state queued to this stage has arrived; raises after timeout_ms
        (the reference polls without a limit, cuda_fused_infer.go:575-591)."""
        self._check(self._lib.mg_wait_mailbox(self._h, timeout_ms), "WaitMailbox")

    def HasMailbox(self) -> bool:
        return True

    def HasL3(self) -> bool:
        return True

    def QueueHiddenToL3(self) -> None:
        """Asynchronous copy of the hidden state to the pinned host buffer on the copy stream
        (cuda_fused_infer.go:686-703)."""
        self._check(self._lib.mg_queue_hidden_to_l3(self._h), "QueueHiddenToL3")

    def WaitL3(self, timeout_ms: int = 1000) -> None:
        self._check(self._lib.mg_wait_l3(self._h, timeout_ms), "WaitL3")

    def GetL3Hidden(self) -> np.ndarray:
        """The pinned host buffer as an array; valid after QueueHiddenToL3 + WaitL3."""
        p = self._lib.mg_l3_hidden(self._h)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(self.cfg.dim,)).copy()

    def ReadHiddenBlocking(self) -> np.ndarray:
        return self.ExportHidden()

    # -- replay API (cuda_graph.go:313-739) -----------------------------------------------------
    def CaptureGraph(self, cfg: GraphCaptureConfig, pos: int = 0):
        """Returns a handle for replaying layers [LayerStart, LayerEnd); None for an unsupported
        StreamCount, like the reference (cuda_graph.go:315-325)."""
        if cfg.StreamCount == 0:
            cfg.StreamCount = 1
        if cfg.StreamCount not in (1, 2):
            return None
        self.BuildFusedDispatch()
        return CUDAGraph(self, cfg)

    def UpdateAndLaunch(self, g: CUDAGraph, pos: int) -> bool:
        """The reference re-captures and patches the executable graph for a new position
        (cuda_graph.go:673-715); here the position is a device-side value, so this is Launch."""
        if not g.captured:
            return False
        g.Launch(pos)
        return True

    def UploadHidden(self, data) -> None:
        self._check(self._lib.mg_upload_hidden(self._h, _host_ptr(np.ascontiguousarray(data, np.float32))),
                    "UploadHidden")

    def ReadHidden(self) -> np.ndarray:
        return self.ExportHidden()

    def ValidateGraphCapture(self, hiddenIn, layerStart: int, layerEnd: int) -> bool:
        """Plain launches against the replay path on the same input at position 0; True when the
        hidden states agree to 1e-3 like the reference's check (cuda_graph.go:554-601)."""
        d = C.c_float(0.0)
        a = np.ascontiguousarray(hiddenIn, np.float32)
        self._check(self._lib.mg_validate_replay(self._h, _np_ptr(a), layerStart, layerEnd, C.byref(d)),
                    "ValidateGraphCapture")
        self.last_validate_diff = float(d.value)
        return bool(d.value < 1e-3)

    def ExportHidden(self) -> np.ndarray:
        out = np.empty(self.cfg.dim, np.float32)
        self._check(self._lib.mg_export_hidden(self._h, _np_ptr(out)), "ExportHidden")
        return out

    def StepToken(self, token: int, pos: int, logitsOut=None) -> int:
        """Greedy step with the tied embedding; returns the argmax token."""
        nxt = C.c_int(-1)
        rc = self._lib.mg_step_token(self._h, int(token), pos, C.byref(nxt), _host_ptr(logitsOut))
        self._check(rc, "StepToken")
        return nxt.value

    def Generate(self, prompt, n_new: int, start_pos: int = 0) -> np.ndarray:
        p = np.ascontiguousarray(prompt, dtype=np.int32)
        out = np.empty(n_new, np.int32)
        rc = self._lib.mg_generate(self._h, _np_ptr(p), p.size, n_new, start_pos, _np_ptr(out))
        self._check(rc, "Generate")
        return out

    def SetCursor(self, token: int, pos: int) -> None:
        self._check(self._lib.mg_set_cursor(self._h, int(token), pos), "SetCursor")

    def GetCursor(self):
        t, p = C.c_int(), C.c_int()
        self._check(self._lib.mg_get_cursor(self._h, C.byref(t), C.byref(p)), "GetCursor")
        return t.value, p.value

    def EnqueueGreedy(self, n_steps: int) -> None:
        self._check(self._lib.mg_enqueue_greedy(self._h, n_steps), "EnqueueGreedy")

    def Sync(self) -> None:
        self._check(self._lib.mg_sync(self._h), "Sync")

    # -- introspection ----------------------------------------------------
    def DequantRows(self, idx: int, row0: int, nrows: int, cols: int) -> np.ndarray:
        out = np.empty((nrows, cols), np.float32)
        self._check(self._lib.mg_dequant_rows(self._h, idx, row0, nrows, _np_ptr(out)), "DequantRows")
        return out

    def ReadKV(self, layer: int, pos0: int, npos: int):
        k = np.empty((npos, self.cfg.kv_dim), np.uint16)
        v = np.empty((npos, self.cfg.kv_dim), np.uint16)
        self._check(self._lib.mg_read_kv(self._h, layer, pos0, npos, _np_ptr(k), _np_ptr(v)), "ReadKV")
        return k, v

    def TraceStep(self) -> np.ndarray:
        """SM-clock stamps [n_ctas, n_events] of one greedy step (see mg_trace_step)."""
        cap = 256 * (self.cfg.n_layers + 1) * 64
        buf = np.zeros(cap, np.int64)
        n_ctas, n_ev = C.c_int(), C.c_int()
        self._check(self._lib.mg_trace_step(self._h, _np_ptr(buf), cap, C.byref(n_ctas), C.byref(n_ev)), "TraceStep")
        return buf[: n_ctas.value * n_ev.value].reshape(n_ctas.value, n_ev.value)

    # -- device memory from the engine's arena (cuda_tensor.go:19-44, gpu_alloc.go:45-241) ----------
    def DeviceAlloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        self._check(self._lib.mg_device_alloc(self._h, nbytes, C.byref(p)), "DeviceAlloc")
        return p.value

    def DeviceFree(self, ptr: int) -> None:
        self._check(self._lib.mg_device_free(self._h, ptr), "DeviceFree")

    def DeviceUpload(self, ptr: int, host: np.ndarray) -> None:
        a = np.ascontiguousarray(host)
        self._check(self._lib.mg_device_upload(self._h, ptr, _np_ptr(a), a.nbytes), "DeviceUpload")

    def DeviceDownload(self, host: np.ndarray, ptr: int) -> None:
        self._check(self._lib.mg_device_download(self._h, _np_ptr(host), ptr, host.nbytes), "DeviceDownload")

    def DeviceZero(self, ptr: int, nbytes: int) -> None:
        self._check(self._lib.mg_device_zero(self._h, ptr, nbytes), "DeviceZero")

    def ArenaStats(self) -> dict:
        t, u, p, lf, o = C.c_size_t(), C.c_size_t(), C.c_size_t(), C.c_size_t(), C.c_int()
        self._check(self._lib.mg_arena_stats(self._h, C.byref(t), C.byref(u), C.byref(p), C.byref(lf), C.byref(o)), "ArenaStats")
        return {"total": t.value, "in_use": u.value, "peak": p.value, "largest_free": lf.value, "outside": o.value}

    def SetWaitLimit(self, ms: int) -> None:
        """Limit of every wait inside the persistent kernel; a wait that runs out makes the step
        raise with MG_ERR_TIMEOUT (the reference's WaitMailbox spins without one)."""
        self._check(self._lib.mg_set_wait_limit_ms(self._h, int(ms)), "SetWaitLimit")

    def DecodePath(self) -> int:
        """Bit 0: persistent kernel; bit 1: its feed-forward block without an exchange of the middle
        vector; bit 2: tensor-parallel exchange inside the kernels (after BuildFusedDispatch)."""
        return self._lib.mg_decode_path(self._h)

    def TpInitAbsentPeers(self, size: int) -> None:
        """Test aid without a counterpart in the reference: make this engine rank 0 of a `size`-rank
        tensor-parallel group whose other ranks do not exist, so the bounded waits inside the
        persistent kernel can be shown to run out on one GPU.  Call before uploading weights."""
        self._check(self._lib.mg_tp_init_absent_peers(self._h, int(size)), "TpInitAbsentPeers")

    @property
    def stream(self) -> int:
        return self._lib.mg_stream(self._h) or 0

    def LaunchCount(self) -> int:
        return int(self._lib.mg_launch_count(self._h))

    def DeviceBytes(self) -> int:
        return int(self._lib.mg_device_bytes(self._h))


def _host_ptr(x):
    if x is None:
        return None
    if isinstance(x, np.ndarray):
        assert x.dtype == np.float32 and x.flags["C_CONTIGUOUS"]
        return _np_ptr(x)
    return C.c_void_p(x.data_ptr())   # torch CPU tensor (pinned or not)
