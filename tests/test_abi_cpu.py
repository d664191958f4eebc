"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "mongoose_kernels.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"MG_API\s+[\w\s\*]+?\b(mongoose_\w+|mg_\w+)\s*\(", text)


def test_header_declares_reference_symbols():
    names = set(declared_symbols())
    # mandatory symbols of tw_load_kernels (kernels.go:224) and the decode hot path
    for n in ("mongoose_rmsnorm", "mongoose_relu", "mongoose_add_inplace", "mongoose_embedding_gather",
              "mongoose_rmsnorm_out", "mongoose_q8_matvec", "mongoose_q4_matvec", "mongoose_q4_0_matvec",
              "mongoose_q4_0_matvec_dp4a", "mongoose_q8_quantize_act", "mongoose_q4_0_matvec_dp4a_preq",
              "mongoose_q4_0_matvec_dp4a_batch", "mongoose_q8_quantize_act_batch", "mongoose_rope",
              "mongoose_kv_cache_write", "mongoose_decode_attention", "mongoose_silu_gate_mul",
              "mongoose_copy", "mongoose_zero", "mongoose_sync", "mongoose_fp32_to_fp16",
              "mongoose_fp16_to_fp32", "mongoose_fused_add_rmsnorm", "mongoose_partial_step_q4_fused_graph"):
        assert n in names, n


def test_library_exports_every_declared_symbol(mglib):
    from mongoose_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 45
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(raw, n), f"{n} is declared in the header but not exported"
        assert n in _lib.SIGNATURES, f"{n} has no ctypes signature"
    assert set(_lib.SIGNATURES) <= set(names), set(_lib.SIGNATURES) - set(names)


def test_version_string(mglib):
    assert b"sm_100a" in mglib.mg_version()


def test_engine_rejects_bad_config_without_gpu(mglib):
    from mongoose_b200 import _lib
    h = ctypes.c_void_p()
    bad = _lib.MgConfig(dim=100, kv_dim=20, head_dim=10, n_heads=10, n_kv_heads=2, ffn_dim=64, vocab=10,
                        n_layers=1, max_seq=8, rope_theta=1e4, rms_eps=0, layer_fmt=0, head_fmt=0, device=0,
                        max_batch=1, flags=0)
    assert mglib.mg_create(ctypes.byref(bad), ctypes.byref(h)) == -1 and not h.value
    assert mglib.mg_create(None, ctypes.byref(h)) == -1
    assert mglib.mg_last_error(None) == b"null engine"


def test_plain_c_loader_resolves_every_symbol(mglib, tmp_path):
    """dlopen + dlsym from C, as the reference's loader does (kernels.go:150-226); also proves the
    public header compiles as C."""
    import shutil
    import subprocess
    from mongoose_b200 import _lib
    cc = shutil.which("gcc") or shutil.which("cc")
    assert cc, "no C compiler"
    exe = tmp_path / "abi_dlopen"
    cuda_inc = "/usr/local/cuda/include"
    subprocess.check_call([cc, "-std=c11", "-Wall", "-Werror", "-I", cuda_inc, "-o", str(exe),
                           os.path.join(ROOT, "tests", "abi_dlopen.c"), "-ldl"])
    out = subprocess.run([str(exe), _lib.LIB_PATH], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stderr
    n = int(out.stdout.split()[0])
    assert n == len(set(declared_symbols())), "abi_dlopen.c must list every symbol the header declares"
