"""dlopen of libmongoose_kernels.so: the Python stand-in for the reference's
``LoadKernels`` / ``tw_load_kernels`` (kernels.go:150-226, 556-591).

There is no fallback: if the library is missing or a symbol does not resolve
the import fails with the reason, as the reference returns -2 when a
mandatory symbol is absent (kernels.go:224).
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmongoose_kernels.so")

vp, ci, cf, cd, sz = C.c_void_p, C.c_int, C.c_float, C.c_double, C.c_size_t


class MgConfig(C.Structure):
    """struct mg_config of include/mongoose_kernels.h."""
    _fields_ = [("dim", ci), ("kv_dim", ci), ("head_dim", ci), ("n_heads", ci), ("n_kv_heads", ci),
                ("ffn_dim", ci), ("vocab", ci), ("n_layers", ci), ("max_seq", ci),
                ("rope_theta", cd), ("rms_eps", cf), ("layer_fmt", ci), ("head_fmt", ci),
                ("device", ci), ("max_batch", ci), ("flags", ci)]


class MgTpShard(C.Structure):
    """struct mg_tp_shard of include/mongoose_kernels.h."""
    _fields_ = [("q_head0", ci), ("q_head1", ci), ("kv_head0", ci), ("kv_head1", ci),
                ("ffn0", ci), ("ffn1", ci), ("vocab0", ci), ("vocab1", ci)]


# name -> (restype, argtypes): every symbol include/mongoose_kernels.h declares.
SIGNATURES = {
    # reference ABI (stream is the last argument everywhere)
    "mongoose_rmsnorm": (None, [vp, vp, ci, ci, vp]),
    "mongoose_rmsnorm_out": (None, [vp, vp, vp, ci, ci, vp]),
    "mongoose_fused_add_rmsnorm": (None, [vp, vp, vp, vp, ci, ci, vp]),
    "mongoose_relu": (None, [vp, ci, vp]),
    "mongoose_add_inplace": (None, [vp, vp, ci, vp]),
    "mongoose_embedding_gather": (None, [vp, vp, vp, vp, ci, ci, vp]),
    "mongoose_embed_gather": (None, [vp, vp, vp, ci, ci, vp]),
    "mongoose_silu_gate_mul": (None, [vp, vp, vp, ci, vp]),
    "mongoose_rope": (None, [vp, vp, vp, ci, ci, ci, ci, vp]),
    "mongoose_kv_cache_write": (None, [vp, vp, ci, ci, vp]),
    "mongoose_decode_attention": (None, [vp, vp, vp, vp, ci, ci, ci, ci, ci, vp]),
    "mongoose_q8_matvec": (None, [vp, vp, vp, vp, ci, ci, vp]),
    "mongoose_q4_matvec": (None, [vp, vp, vp, vp, ci, ci, vp]),
    "mongoose_q4_0_matvec": (None, [vp, vp, vp, ci, ci, vp]),
    "mongoose_q8_0_matvec": (None, [vp, vp, vp, ci, ci, vp]),
    "mongoose_q8_quantize_act": (None, [vp, vp, ci, vp]),
    "mongoose_q8_quantize_act_batch": (None, [vp, vp, ci, ci, vp]),
    "mongoose_q4_0_matvec_dp4a": (None, [vp, vp, vp, ci, ci, vp, vp]),
    "mongoose_q4_0_matvec_dp4a_preq": (None, [vp, vp, vp, ci, ci, vp]),
    "mongoose_q4_0_matvec_dp4a_batch": (None, [vp, vp, vp, ci, ci, ci, vp]),
    "mongoose_q4_0_matvec_dp4a_static": (ci, [vp, vp, vp, ci, ci, vp]),
    "mongoose_static_scratch_error": (C.c_char_p, []),
    "mongoose_copy": (None, [vp, vp, sz, vp]),
    "mongoose_zero": (None, [vp, sz, vp]),
    "mongoose_sync": (None, [vp]),
    "mongoose_fp32_to_fp16": (None, [vp, vp, ci, vp]),
    "mongoose_fp16_to_fp32": (None, [vp, vp, ci, vp]),
    "mongoose_partial_step_q4_fused_graph": (None, [vp] * 25 + [ci] * 10 + [vp]),
    # engine
    "mg_create": (ci, [C.POINTER(MgConfig), C.POINTER(vp)]),
    "mg_destroy": (None, [vp]),
    "mg_num_weights": (ci, [vp]),
    "mg_set_weight": (ci, [vp, ci, vp, sz]),
    "mg_set_weight_raw": (ci, [vp, ci, vp, sz, ci]),
    "mg_build": (ci, [vp]),
    "mg_reset_kv": (ci, [vp]),
    "mg_partial_step": (ci, [vp, vp, ci, ci, ci, vp, vp]),
    "mg_export_hidden": (ci, [vp, vp]),
    "mg_step_token": (ci, [vp, ci, ci, vp, vp]),
    "mg_generate": (ci, [vp, vp, ci, ci, ci, vp]),
    "mg_enqueue_greedy": (ci, [vp, ci]),
    "mg_set_cursor": (ci, [vp, ci, ci]),
    "mg_get_cursor": (ci, [vp, vp, vp]),
    "mg_sync": (ci, [vp]),
    "mg_dequant_rows": (ci, [vp, ci, ci, ci, vp]),
    "mg_read_kv": (ci, [vp, ci, ci, ci, vp, vp]),
    "mg_trace_step": (ci, [vp, vp, ci, vp, vp]),
    "mg_set_wait_limit_ms": (ci, [vp, ci]),
    "mg_decode_path": (ci, [vp]),
    "mg_tp_init_absent_peers": (ci, [vp, ci]),
    "mg_device_alloc": (ci, [vp, C.c_size_t, C.POINTER(vp)]),
    "mg_device_free": (ci, [vp, vp]),
    "mg_device_upload": (ci, [vp, vp, vp, C.c_size_t]),
    "mg_device_download": (ci, [vp, vp, vp, C.c_size_t]),
    "mg_device_zero": (ci, [vp, vp, C.c_size_t]),
    "mg_arena_stats": (ci, [vp, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.POINTER(C.c_size_t), C.POINTER(ci)]),
    "mg_step_layer_resident": (ci, [vp, ci, ci, vp, vp, vp, vp]),
    "mg_set_vnode_count": (ci, [vp, ci]),
    "mg_vnode_count": (ci, [vp]),
    "mg_record_stage_done": (ci, [vp]),
    "mg_wait_stage_done": (ci, [vp]),
    "mg_sync_stream1": (ci, [vp]),
    "mg_partial_step_continue_on_stream1": (ci, [vp, ci, ci, ci, vp]),
    "mg_queue_hidden_to_l3_on_stream1": (ci, [vp]),
    "mg_set_layer_range": (ci, [vp, ci, ci]),
    "mg_partial_step_continue": (ci, [vp, ci, ci, ci, vp, vp]),
    "mg_queue_hidden_to": (ci, [vp, vp]),
    "mg_wait_mailbox": (ci, [vp, ci]),
    "mg_queue_hidden_to_l3": (ci, [vp]),
    "mg_wait_l3": (ci, [vp, ci]),
    "mg_l3_hidden": (vp, [vp]),
    "mg_upload_hidden": (ci, [vp, vp]),
    "mg_graph_launch": (ci, [vp, ci, ci, ci]),
    "mg_validate_replay": (ci, [vp, vp, ci, ci, vp]),
    "mg_tp_partition": (ci, [vp, ci, ci, vp]),
    "mg_tp_unique_id": (ci, [vp, sz]),
    "mg_tp_init": (ci, [vp, ci, ci, vp, sz]),
    "mg_stream": (vp, [vp]),
    "mg_launch_count": (C.c_longlong, [vp]),
    "mg_device_bytes": (sz, [vp]),
    "mg_last_error": (C.c_char_p, [vp]),
    "mg_version": (C.c_char_p, []),
}

_lib = None


def load(path: str | None = None) -> C.CDLL:
    """Open the library and bind every declared symbol.  Raises with the
    reason when the file is absent or a symbol is missing."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise RuntimeError(
            f"{p} not found: build it with `python -m mongoose_b200.build` "
            "(there is no CPU or PyTorch fallback for this path)")
    lib = C.CDLL(p, mode=C.RTLD_GLOBAL)
    missing = []
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            missing.append(name)
            continue
        fn.restype, fn.argtypes = res, args
    if missing:
        raise RuntimeError(f"{p} does not export: {', '.join(missing)}")
    if path is None:
        _lib = lib
    return lib
