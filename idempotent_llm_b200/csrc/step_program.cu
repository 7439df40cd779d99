// A step of a model as data: a list of kernel calls with their constant arguments (weights, sizes,
// cache entries), run for one step's tokens by ONE call from the host.
//
// The host side of a step is otherwise some two hundred calls through the Python binding, each with
// its checks and its output tensor: 12-15 us apiece, which is what a prompt of up to a thousand tokens
// costs however fast the kernels are.  Here the calls that never change are written down once, when a
// model is put together (parts emit their calls), and a step supplies only what a step brings: its
// packed tokens, the addresses of its buffers and the plan of its attention tiles.  The entry points
// called are the library's own, with the arguments the binding would give them: the same kernels on
// the same numbers, so the same bits.
//
// The reference runs its layers from Python and captures single-token steps into a graph
// (src/detllm/graphed.py:43-73); it has no counterpart of this file.
#include "common.cuh"
#include "step_program.h"

#include <stddef.h>

extern "C" int idm_embed(const int*, const void*, float*, int, int, cudaStream_t);
extern "C" int idm_add_rmsnorm(float*, const float*, int, long long, const float*, float, void*, const int*, int, int,
                               cudaStream_t);
extern "C" int idm_rope_table(const int*, const double*, float*, float*, int, int, cudaStream_t);
extern "C" int idm_gemm_bf16(const void*, const void*, float*, int, int, int, cudaStream_t);
extern "C" int idm_gemm_bf16_residual(const void*, const void*, float*, int, int, int, cudaStream_t);
extern "C" int idm_gemm_bf16_swiglu(const void*, const void*, void*, int, int, int, cudaStream_t);
extern "C" int idm_gemm_bf16_qkv(const void*, const void*, int, int, int, int, int, const float*, const float*, float,
                                 const float*, const float*, void*, void*, void*, void*, void*, const int*, int, int,
                                 const int*, const int*, const int*, cudaStream_t);
extern "C" int idm_attention_tc(const void*, void*, const void*, const void*, int, const int*, int, const int*,
                                const int*, int, const int*, const int*, const int*, const int*, int, int, int, int,
                                float, int, int, int, float*, const int*, int, int, cudaStream_t);

// sizes and offsets of the two records, for the binding to compare with its own definitions
extern "C" int idm_program_layout(int* out) {
    int n = 0;
    out[n++] = (int)sizeof(IdmOp);
    out[n++] = (int)offsetof(IdmOp, i);
    out[n++] = (int)offsetof(IdmOp, f);
    out[n++] = (int)offsetof(IdmOp, p);
    out[n++] = (int)sizeof(IdmAttnPlan);
    out[n++] = (int)offsetof(IdmAttnPlan, n_tiles);
    out[n++] = (int)sizeof(IdmStep);
    out[n++] = (int)offsetof(IdmStep, buf);
    out[n++] = (int)offsetof(IdmStep, attn);
    out[n++] = (int)offsetof(IdmStep, n_tokens);
    out[n++] = IDM_PROGRAM_BUFFERS;
    out[n++] = IDM_PROGRAM_PLANS;
    return n;
}

#define BUF(k) (st->buf[(k)])

// Runs `ops` for the step `st`; returns 0, or non-zero with the message of the call that refused
// (idm_last_error) and its place in st->failed_op.  st->launches counts the kernels launched.
extern "C" int idm_run_program(const IdmOp* ops, int n_ops, IdmStep* st, cudaStream_t stream) {
    const int n = st->n_tokens, rows = st->n_rows;
    st->launches = 0;
    st->failed_op = -1;
    if (n <= 0) return 0;
    for (int k = 0; k < n_ops; ++k) {
        const IdmOp& o = ops[k];
        const int* i = o.i;
        int rc = 0, launched = 1;
        switch (o.kind) {
        case IDM_OP_EMBED:
            rc = idm_embed(st->tokens, o.p[0], (float*)BUF(i[1]), n, i[0], stream);
            break;
        case IDM_OP_ROPE_TABLE:
            // steps of many tokens also get the table with the tokens of one dim side by side (what the
            // q/k/v product's epilogue of such steps reads)
            rc = idm_rope_table(st->positions, (const double*)o.p[0], (float*)BUF(i[1]),
                                n > 64 ? (float*)BUF(i[2]) : nullptr, n, i[0], stream);
            break;
        case IDM_OP_ADD_RMSNORM: {
            const int n_out = i[3] ? rows : n;
            launched = n_out > 0;
            rc = idm_add_rmsnorm((float*)BUF(i[1]), nullptr, 0, 0, (const float*)o.p[0], o.f[0], BUF(i[2]),
                                 i[3] ? st->rows : nullptr, n_out, i[0], stream);
            break;
        }
        case IDM_OP_GEMM_QKV:
            rc = idm_gemm_bf16_qkv(BUF(i[4]), o.p[0], n, i[0], i[1], i[2], i[3], (const float*)o.p[1],
                                   (const float*)o.p[2], o.f[0], i[6] >= 0 ? (const float*)BUF(i[6]) : nullptr,
                                   (i[6] >= 0 && n > 64) ? (const float*)BUF(i[7]) : nullptr, BUF(i[5]), nullptr, nullptr,
                                   (void*)o.p[3], (void*)o.p[4], (const int*)o.p[5], i[8], i[9], st->token_seq,
                                   st->positions, st->slots, stream);
            break;
        case IDM_OP_ATTENTION: {
            const IdmAttnPlan& a = st->attn[i[7]];
            launched = a.n_tiles > 0;
            rc = idm_attention_tc(BUF(i[5]), BUF(i[6]), o.p[0], o.p[1], i[0], (const int*)o.p[2], i[1], a.tile_seq,
                                  a.tile_start, a.n_tiles, st->cu_q, st->q_start, st->kv_len, st->slots, n, i[2], i[3],
                                  i[4], o.f[0], a.run_blocks, a.max_runs, a.rows_cap, a.scratch, a.tile_pool,
                                  a.max_parts, a.runs_per_part, stream);
            break;
        }
        case IDM_OP_GEMM_RESIDUAL:
            rc = idm_gemm_bf16_residual(BUF(i[2]), o.p[0], (float*)BUF(i[3]), n, i[0], i[1], stream);
            break;
        case IDM_OP_GEMM_SWIGLU:
            rc = idm_gemm_bf16_swiglu(BUF(i[2]), o.p[0], BUF(i[3]), n, i[0], i[1], stream);
            break;
        case IDM_OP_GEMM_STORE: {
            const int m = i[4] ? rows : n;
            launched = m > 0;
            if (m > 0) rc = idm_gemm_bf16(BUF(i[2]), o.p[0], (float*)BUF(i[3]), m, i[0], i[1], stream);
            break;
        }
        default:
            rc = idm_fail("program: call %d has the unknown kind %d", k, o.kind);
        }
        if (rc != 0) {
            st->failed_op = k;
            return rc;
        }
        st->launches += launched;
    }
    return 0;
}
