/* Resolves the library's symbols the way the reference's loader does (dlopen + dlsym by name,
 * kernels.go:150-226), compiled as C against the public header so that the header itself is checked
 * to be valid C.  Needs no GPU: it calls only mg_version, mg_tp_partition and the argument checks of
 * mg_create.  Usage: abi_dlopen <path to libmongoose_kernels.so>; prints the number of symbols
 * resolved, exits non-zero on the first one missing. */
#include <dlfcn.h>
#include <stdio.h>
#include <string.h>

#include "../include/mongoose_kernels.h"

static const char* kNames[] = {
    "mongoose_rmsnorm", "mongoose_rmsnorm_out", "mongoose_fused_add_rmsnorm", "mongoose_relu",
    "mongoose_add_inplace", "mongoose_embedding_gather", "mongoose_silu_gate_mul", "mongoose_rope",
    "mongoose_kv_cache_write", "mongoose_decode_attention", "mongoose_q8_matvec", "mongoose_q4_matvec",
    "mongoose_q4_0_matvec", "mongoose_q8_0_matvec", "mongoose_q8_quantize_act", "mongoose_q4_0_matvec_dp4a",
    "mongoose_q4_0_matvec_dp4a_preq", "mongoose_q4_0_matvec_dp4a_batch", "mongoose_q8_quantize_act_batch",
    "mongoose_copy", "mongoose_zero", "mongoose_sync", "mongoose_fp32_to_fp16", "mongoose_fp16_to_fp32",
    "mongoose_partial_step_q4_fused_graph", "mongoose_q4_0_matvec_dp4a_static", "mongoose_static_scratch_error",
    "mongoose_embed_gather",
    "mg_create", "mg_destroy", "mg_num_weights", "mg_set_weight", "mg_set_weight_raw", "mg_build",
    "mg_reset_kv", "mg_partial_step", "mg_partial_step_continue", "mg_export_hidden", "mg_step_token",
    "mg_generate", "mg_enqueue_greedy", "mg_set_cursor", "mg_get_cursor", "mg_sync", "mg_dequant_rows",
    "mg_read_kv", "mg_trace_step", "mg_set_wait_limit_ms", "mg_decode_path", "mg_tp_init_absent_peers", "mg_device_alloc", "mg_device_free", "mg_device_upload",
    "mg_device_download", "mg_device_zero", "mg_arena_stats", "mg_step_layer_resident", "mg_set_vnode_count",
    "mg_vnode_count", "mg_record_stage_done", "mg_wait_stage_done", "mg_sync_stream1",
    "mg_partial_step_continue_on_stream1", "mg_queue_hidden_to_l3_on_stream1", "mg_upload_hidden", "mg_graph_launch", "mg_validate_replay",
    "mg_set_layer_range", "mg_queue_hidden_to", "mg_wait_mailbox", "mg_queue_hidden_to_l3", "mg_wait_l3",
    "mg_l3_hidden", "mg_tp_partition", "mg_tp_unique_id", "mg_tp_init", "mg_stream", "mg_launch_count",
    "mg_device_bytes", "mg_last_error", "mg_version",
};

typedef const char* (*version_fn)(void);
typedef int (*create_fn)(const mg_config*, mg_engine**);
typedef int (*partition_fn)(const mg_config*, int, int, mg_tp_shard*);

int main(int argc, char** argv) {
    if (argc < 2) {
        fprintf(stderr, "usage: %s libmongoose_kernels.so\n", argv[0]);
        return 2;
    }
    void* lib = dlopen(argv[1], RTLD_NOW | RTLD_LOCAL);
    if (!lib) {
        fprintf(stderr, "dlopen: %s\n", dlerror());
        return 1;
    }
    const int n = (int)(sizeof kNames / sizeof kNames[0]);
    for (int i = 0; i < n; i++)
        if (!dlsym(lib, kNames[i])) {
            fprintf(stderr, "missing symbol: %s\n", kNames[i]);
            return 1;
        }
    version_fn version = (version_fn)dlsym(lib, "mg_version");
    if (!strstr(version(), "sm_100a")) return 1;

    /* argument checks run before any CUDA call */
    mg_config bad;
    memset(&bad, 0, sizeof bad);
    mg_engine* e = (mg_engine*)0x1;
    if (((create_fn)dlsym(lib, "mg_create"))(&bad, &e) != MG_ERR_ARG || e != NULL) return 1;

    /* 28 query heads on 4 KV heads over 8 ranks: pairs of ranks share a KV head, 4 + 3 query heads */
    mg_config c;
    memset(&c, 0, sizeof c);
    c.dim = 3584; c.kv_dim = 512; c.head_dim = 128; c.n_heads = 28; c.n_kv_heads = 4;
    c.ffn_dim = 18944; c.vocab = 152064; c.n_layers = 28; c.max_seq = 512;
    mg_tp_shard s;
    partition_fn part = (partition_fn)dlsym(lib, "mg_tp_partition");
    if (part(&c, 1, 8, &s) != MG_OK) return 1;
    if (s.q_head0 != 4 || s.q_head1 != 7 || s.kv_head0 != 0 || s.kv_head1 != 1) return 1;
    if (s.ffn0 != 2368 || s.ffn1 != 4736 || s.vocab0 != 19008 || s.vocab1 != 38016) return 1;
    if (part(&c, 0, 3, &s) != MG_ERR_UNSUPPORTED) return 1;

    printf("%d symbols resolved\n", n);
    dlclose(lib);
    return 0;
}
