// The native step executor: what one model step does on the host, in one call.
//
// tamnd/fastmlx's engine loop is compiled code on one goroutine (enginecore/core.go:134-171 drains
// submissions and steps the scheduler, scheduler/scheduler.go:126-154 runs one model step); a
// Python loop that makes a hundred and more kernel launches per step through ctypes spends about
// 15 us of host time on each, which bounds every step that is not a replayed CUDA graph.  Here
// the parts of a model describe themselves once, at load time, as a short program over numbered
// activation buffers ("registers"); per step the executor lays the batch out (tokens, positions,
// rows, block tables and slot mappings in one packed buffer, one host-to-device copy) and walks the
// program, choosing for each operation the kernel its row count calls for, exactly as the
// Python path chooses (kernels/__init__.py: linear, paged_attention).  The kernels themselves are
// those of the other libraries: the loader hands their entry points over as a table.
//
// The structures below are mirrored field by field in engine/native.py (ctypes).
#pragma once
#include <cuda_runtime.h>

#define FMX_MAX_GROUPS 8

enum FmxOpKind {
  FMX_OP_EMBED = 0,        // out0[T, cols] = table w[ids]; ids = the step's tokens
  FMX_OP_ADD_RMSNORM = 1,  // out0 = norm(stream (+ in0)) * vec; in1 = the stream register (-1: in0 is the stream's first value)
  FMX_OP_LINEAR = 2,       // out0 = in0 . w^T (+ bias); out0 = -2: the step's logits
  FMX_OP_GATE_UP = 3,      // out0[rows, n/2] = silu(gate) * up of in0 . w^T; out1 = a register of n columns for the unfused route
  FMX_OP_ATTENTION = 4,    // out0[T, nh*hd] = attention of in0 (q | k | v) over the layer's pages; rotates and stores first
  FMX_OP_GATHER_ROWS = 5,  // out0[wanted, cols] = in0[wanted rows]
};

struct FmxReg {
  int cols;
  int dtype;               // FMX_F32 / FMX_BF16
};

struct FmxOp {
  int kind;
  int in0, in1, out0, out1;
  int wanted_rows;         // 0: the op runs over all T tokens; 1: over the wanted rows only
  const void* w;           // matrix [n, k] (embedding: [table_rows, n])
  const float* bias;       // 32-bit, or null
  const float* vec;        // norm weight, or the rotary inverse frequencies
  int w_dtype;
  long long ldw;
  int n, k;
  int out_dtype;
  int block;               // gate/up rows alternate in blocks of this many (0: all gates, then all ups)
  float eps, scale;
  long long table_rows;
  int init;                // ADD_RMSNORM: in0 is the stream's first value, written into in1 (a 32-bit stream beside bfloat16)
  // attention
  int nh, nkv, hd, window, rot, trad, store, group, share_kv;   // store: this layer writes k and v; share_kv: the input holds queries only
  void* kv;                // the layer's pages [num_pages, 2, nkv, page_size, hd]
  int page_size;
  long long num_pages;
  void* fn_attn_decode;    // entry points of the attention library of this head size (null: none for this size or type)
  void* fn_attn_prefill;
  void* fn_attn_prefill_tc;
  void* fn_attn_plan;
  void* fn_attn_prefill_tc_plan;   // how many CTAs share the keys of a pair of query tiles
  int tc_attention_ok;     // sizes the tensor-memory attention kernel takes (head size, heads per kv head, page size, no window)
};

// Entry points of the other libraries (kernels/lib.py loads them); null where a library is absent.
struct FmxKernelTable {
  void* gather_rows;
  void* gather_rows_f32_to_bf16;
  void* add_rmsnorm;
  void* silu_mul;
  void* gemm_simple;
  void* rope_kv_write;
  void* paged_attention_simple;
  void* fill_rows;
  void* gemv;
  void* gemm_tcgen05;
  void* gemm_tcgen05_plan_fills;
  void* gemv_argmax;
};

// One laid-out step: device pointers into the packed buffer, and the step's workspaces.
struct FmxStepDesc {
  int T, R, n_want, max_q_len, max_ctx_after, all_decode, n_splits, n_groups;
  // a mixed step whose first rows bring one token each: how many, the longest context among them after the step, and
  // the longest portion and the longest context after the step among the rows behind them; all 0 where the step is not
  // mixed so
  int decode_rows, decode_max_ctx, rest_max_q_len, rest_max_ctx;
  const int* tokens;
  const int* positions;
  const int* token_row;
  const int* row_start;
  const int* row_ctx;
  const int* row_slot;
  const int* want;
  const int* block_tables[FMX_MAX_GROUPS];
  int bt_stride[FMX_MAX_GROUPS];
  const long long* slot_mapping[FMX_MAX_GROUPS];
  int* status;
  void* arena;
  long long arena_bytes;
  float* logits;
  float* attn_scratch;
  long long attn_scratch_floats;
  int* attn_tickets;
  int attn_tickets_n;
  // not null: the head chooses greedily inside its product (at most 16 wanted rows, bfloat16 operands) and
  // leaves ids here instead of logits; greedy_best / greedy_ticket are that kernel's words, zero between launches
  int* greedy_ids;
  void* greedy_best;
  int* greedy_ticket;
};

// What the caller knows of a step before it is laid out: one entry per request.
struct FmxBatchIn {
  int R;
  const int* q_lens;       // [R] tokens each request brings
  const int* ctx_lens;     // [R] tokens already in its cache
  const int* slots;        // [R] its state slot = its row in the block-table mirrors
  const int* tokens;       // [sum q_lens]
  int n_want;
  const int* want;         // [n_want] indices among the step's tokens
  int pad_rows, pad_blocks;
  int page_size, n_groups;
  const int* mirror[FMX_MAX_GROUPS];      // block tables by slot, [slots, mirror_cols], -1 where there is no page
  int mirror_cols[FMX_MAX_GROUPS];
};

extern "C" {
void* fmx_exec_create(const FmxOp* ops, int n_ops, const FmxReg* regs, int n_regs, const FmxKernelTable* kernels,
                      int sms, const char* cublas_path, void* cublas_workspace, long long cublas_workspace_bytes);
void fmx_exec_destroy(void* exec);
// Bytes of arena a step of T tokens needs.
long long fmx_exec_arena_bytes(void* exec, int T);
// Ints of packed buffer a step needs (a multiple of 4).
long long fmx_exec_layout_ints(const FmxBatchIn* in);
// Lay the step out into `host` (>= fmx_exec_layout_ints ints, pinned), copy it to `dev` on the stream and fill the
// pointers of `desc` (T, R, n_want, the sizes and every array); workspaces, arena, logits and status are the caller's.
// dev == null: nothing is copied and the pointers of `desc` point into `host` (how the layout is tested without a GPU).
int fmx_exec_layout(const FmxBatchIn* in, int* host, int* dev, long long capacity_ints, FmxStepDesc* desc,
                    cudaStream_t stream);
// Run the program over a laid-out step.  -> 0, or non-zero after leaving a text for fmx_last_error().
int fmx_exec_forward(void* exec, const FmxStepDesc* desc, cudaStream_t stream);
// Kernel entry calls made by this executor so far.
long long fmx_exec_launches(void* exec);
}
