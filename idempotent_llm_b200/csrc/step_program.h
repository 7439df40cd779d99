// The records of a step program (step_program.cu): a call with its constant arguments, and what a step
// supplies.  The Python binding defines the same records (kernels/program.py) and compares sizes and
// offsets with idm_program_layout() when it loads the library.
#pragma once

#define IDM_OP_INTS 10
#define IDM_OP_FLOATS 2
#define IDM_OP_POINTERS 6
#define IDM_PROGRAM_BUFFERS 16
#define IDM_PROGRAM_PLANS 4

enum IdmOpKind {
    IDM_OP_EMBED = 0,         // buf[i1] <- table p0 [vocab, i0] rows of the step's tokens, 32-bit
    IDM_OP_ROPE_TABLE = 1,    // buf[i1] (and buf[i2] with more than 64 tokens) <- cos/sin of positions x inv_freq p0 [i0]
    IDM_OP_ADD_RMSNORM = 2,   // buf[i2] <- norm(buf[i1]) with weight p0 [i0], eps f0; i3: only the step's wanted rows
    IDM_OP_GEMM_QKV = 3,      // x buf[i4] . w p0 [(i1 + 2 i2) i3, i0]; q/k norm p1, p2 (eps f0), rotation by buf[i6] / buf[i7],
                              // q to buf[i5], k and v to the cache entry (p3, p4, table p5 with i8 entries a slot, ring i9)
    IDM_OP_ATTENTION = 4,     // buf[i6] <- attention of q buf[i5] over the cache entry (p0, p1; i0 pages; table p2, i1 entries
                              // a slot); heads i2 / i3 of size i4, scale f0; tiles and scratch from the step's plan i7
    IDM_OP_GEMM_RESIDUAL = 5, // buf[i3] += buf[i2] . w p0 [i0, i1]
    IDM_OP_GEMM_SWIGLU = 6,   // buf[i3] <- silu(gate) * up of buf[i2] . w p0 (tiled gate/up rows of i0 features, inner size i1)
    IDM_OP_GEMM_STORE = 7,    // buf[i3] <- buf[i2] . w p0 [i0, i1] in 32-bit; i4: the rows are the step's wanted rows
};

struct IdmOp {
    int kind;
    int i[IDM_OP_INTS];
    float f[IDM_OP_FLOATS];
    int pad;
    const void* p[IDM_OP_POINTERS];
};

// The tiles of a step's attention for one arrangement of heads (what every layer with these heads shares)
struct IdmAttnPlan {
    const int* tile_seq;
    const int* tile_start;
    const int* tile_pool;
    float* scratch;
    int n_tiles, rows_cap, max_runs, max_parts, runs_per_part, run_blocks;
};

struct IdmStep {
    const int *tokens, *token_seq, *positions, *cu_q, *slots, *q_start, *kv_len, *rows;
    void* buf[IDM_PROGRAM_BUFFERS];
    IdmAttnPlan attn[IDM_PROGRAM_PLANS];
    int n_tokens, n_rows;      // tokens of the step; rows whose logits are wanted
    int launches, failed_op;   // out: kernels launched; the call that refused (-1: none)
};
