// Host code only: the step executor described in step_executor.h.  It owns no kernel; it calls
// the entry points of the other libraries and, for the matrix products that go to the library
// (where tamnd/fastmlx calls its library's matmul, compute/models/qwen3_forward.go:111-115),
// cuBLAS through a handle of its own with a workspace that the caller provides.
#include <cublas_v2.h>
#include <dlfcn.h>
#include <stdint.h>
#include <string.h>

#include <vector>

#include "common.cuh"
#include "step_executor.h"

namespace {
// ---- entry points of the kernel libraries, by their C signatures
typedef int (*gather_rows_fn)(const void*, const int*, void*, int, int, long long, int, int*, int, cudaStream_t);
typedef int (*gather_rows_f32_to_bf16_fn)(const float*, const int*, void*, int, int, long long, int*, int, cudaStream_t);
typedef int (*add_rmsnorm_fn)(const void*, void*, const float*, void*, int, int, float, int, int, int, cudaStream_t);
typedef int (*silu_mul_fn)(const void*, void*, int, int, int, int, cudaStream_t);
typedef int (*gemm_simple_fn)(const void*, const void*, const float*, void*, int, int, int, long long, long long,
                              long long, int, int, int, cudaStream_t);
typedef int (*rope_kv_write_fn)(void*, const int*, const float*, const long long*, void*, int, int, int, int, int, int,
                                int, long long, long long, int, int*, cudaStream_t);
typedef int (*attention_simple_fn)(const void*, long long, const void*, const int*, int, const int*, const int*, void*,
                                   int, int, int, int, int, long long, float, int, int, int, int*, cudaStream_t);
typedef int (*fill_rows_fn)(const float*, void*, int, int, long long, int, cudaStream_t);
typedef int (*gemv_fn)(const void*, long long, const void*, long long, const float*, const void*, long long, void*,
                       long long, int, int, int, int, int, int, int, cudaStream_t);
typedef int (*gemm_tcgen05_fn)(const void*, long long, const void*, long long, void*, long long, const void*, long long,
                               int, int, int, int, int, int, int*, cudaStream_t);
typedef int (*plan_fills_fn)(int, int, int);
typedef int (*attn_decode_fn)(const void*, long long, const void*, const int*, int, const int*, const int*, void*,
                              float*, long long, int*, int, int, int, int, int, long long, float, int, int*,
                              const float*, int, int, int, cudaStream_t);
typedef int (*attn_prefill_fn)(const void*, long long, const void*, const int*, int, const int*, const int*, void*, int,
                               int, int, int, int, long long, float, int, int*, cudaStream_t);
typedef int (*attn_prefill_tc_fn)(const void*, long long, int, const void*, const int*, int, const int*, const int*,
                                  void*, int, int, int, int, int, long long, float, int, int*, int, float*, long long,
                                  cudaStream_t);
typedef int (*attn_plan_fn)(int, int, long long, int);
typedef int (*attn_prefill_tc_plan_fn)(int, int, int, int, int, int);
typedef int (*gemv_argmax_fn)(const void*, long long, const void*, long long, int*, void*, int*, int, int, int, cudaStream_t);

constexpr int GEMV_MAX_ROWS = 16;            // as kernels/__init__.py names them
constexpr int LIBRARY_MIN_FEATURES = 65536;
constexpr int TC_MIN_ROWS = 128;
constexpr int TC_ATTN_MIN_TOKENS = 64;
constexpr int EPI_PLAIN = 0, EPI_SILU_MUL = 1;
constexpr int BAD_TOKEN = 1, BAD_ROW = 4;

// ---- cuBLAS, found at run time in the process (the copy PyTorch has loaded) or by path
struct Cublas {
  void* lib = nullptr;
  cublasHandle_t handle = nullptr;
  cublasStatus_t (*create)(cublasHandle_t*) = nullptr;
  cublasStatus_t (*destroy)(cublasHandle_t) = nullptr;
  cublasStatus_t (*set_stream)(cublasHandle_t, cudaStream_t) = nullptr;
  cublasStatus_t (*set_workspace)(cublasHandle_t, void*, size_t) = nullptr;
  cublasStatus_t (*gemm_ex)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void*, const void*,
                            cudaDataType, int, const void*, cudaDataType, int, const void*, void*, cudaDataType, int,
                            cublasComputeType_t, cublasGemmAlgo_t) = nullptr;
  cudaStream_t stream = (cudaStream_t)-1;

  int open(const char* path, void* workspace, long long workspace_bytes) {
    lib = dlopen("libcublas.so.12", RTLD_NOW | RTLD_NOLOAD);
    if (lib == nullptr && path != nullptr && path[0]) lib = dlopen(path, RTLD_NOW);
    if (lib == nullptr) lib = dlopen("libcublas.so.12", RTLD_NOW);
    if (lib == nullptr) lib = dlopen("libcublas.so", RTLD_NOW);
    if (lib == nullptr) return fmx_fail("the step executor found no cuBLAS library: %s", dlerror());
    *(void**)&create = dlsym(lib, "cublasCreate_v2");
    *(void**)&destroy = dlsym(lib, "cublasDestroy_v2");
    *(void**)&set_stream = dlsym(lib, "cublasSetStream_v2");
    *(void**)&set_workspace = dlsym(lib, "cublasSetWorkspace_v2");
    *(void**)&gemm_ex = dlsym(lib, "cublasGemmEx");
    if (!create || !destroy || !set_stream || !set_workspace || !gemm_ex)
      return fmx_fail("the cuBLAS library lacks an entry point the step executor needs");
    cublasStatus_t st = create(&handle);
    if (st != CUBLAS_STATUS_SUCCESS) return fmx_fail("cublasCreate failed with status %d", (int)st);
    // a workspace of the caller's: the library then allocates nothing, also under stream capture
    if (workspace != nullptr && workspace_bytes > 0) {
      st = set_workspace(handle, workspace, (size_t)workspace_bytes);
      if (st != CUBLAS_STATUS_SUCCESS) return fmx_fail("cublasSetWorkspace failed with status %d", (int)st);
    }
    return 0;
  }
  void close() {
    if (handle != nullptr && destroy != nullptr) destroy(handle);
    handle = nullptr;
  }
  // out[M, N] (row-major, leading dimension ldo) = beta * out + x[M, K] . w[N, K]^T, summed in 32-bit
  int product(const void* x, long long ldx, const void* w, long long ldw, void* out, long long ldo, int out_dtype,
              int M, int N, int K, float beta, cudaStream_t s) {
    if (s != stream) {
      cublasStatus_t st = set_stream(handle, s);
      if (st != CUBLAS_STATUS_SUCCESS) return fmx_fail("cublasSetStream failed with status %d", (int)st);
      stream = s;
    }
    const float alpha = 1.0f;
    cublasStatus_t st = gemm_ex(handle, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, w, CUDA_R_16BF, (int)ldw, x,
                                CUDA_R_16BF, (int)ldx, &beta, out, out_dtype == FMX_F32 ? CUDA_R_32F : CUDA_R_16BF,
                                (int)ldo, CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    if (st != CUBLAS_STATUS_SUCCESS) return fmx_fail("cublasGemmEx failed with status %d (M=%d N=%d K=%d)", (int)st, M, N, K);
    return 0;
  }
};

struct Executor {
  std::vector<FmxOp> ops;
  std::vector<FmxReg> regs;
  FmxKernelTable k;
  int sms;
  Cublas blas;
  bool blas_open = false;
  const char* blas_path = nullptr;
  std::vector<char> blas_path_store;
  void* blas_ws;
  long long blas_ws_bytes;
  long long launches = 0;
  std::vector<long long> offsets;      // per register, for the step being run
};

inline long long align_up(long long v, long long a) { return (v + a - 1) / a * a; }
inline long long elem_size(int dtype) { return dtype == FMX_F32 ? 4 : 2; }

// Where each register of a step of T tokens lies in the arena; -> bytes needed.
long long place_registers(const Executor& ex, int T, std::vector<long long>* offsets) {
  long long at = 0;
  if (offsets != nullptr) offsets->resize(ex.regs.size());
  for (size_t r = 0; r < ex.regs.size(); ++r) {
    at = align_up(at, 256);
    if (offsets != nullptr) (*offsets)[r] = at;
    at += (long long)T * ex.regs[r].cols * elem_size(ex.regs[r].dtype);
  }
  return align_up(at, 256);
}
}  // namespace

namespace {
struct Run {
  Executor& ex;
  const FmxStepDesc& d;
  cudaStream_t stream;

  void* reg(int r) const { return r < 0 ? nullptr : (char*)d.arena + ex.offsets[r]; }
  int rows_of(const FmxOp& op) const { return op.wanted_rows ? d.n_want : d.T; }

  static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }
  // bfloat16 operands laid out as the tensor-core kernels read them (16-byte rows)
  static bool bf16_operands(const void* x, int x_dtype, long long ldx, const void* w, int w_dtype, long long ldw, int M,
                            int K) {
    return x_dtype == FMX_BF16 && w_dtype == FMX_BF16 && M > 0 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 &&
           aligned16(x) && aligned16(w);
  }
  bool fills(int M, int N) const {
    return ex.k.gemm_tcgen05_plan_fills != nullptr && ((plan_fills_fn)ex.k.gemm_tcgen05_plan_fills)(M, N, ex.sms) != 0;
  }

  int library_product(const void* x, long long ldx, const void* w, long long ldw, void* out, long long ldo, int out_dtype,
                      int M, int N, int K, float beta) {
    if (!ex.blas_open) {
      if (ex.blas.open(ex.blas_path, ex.blas_ws, ex.blas_ws_bytes) != 0) return 1;
      ex.blas_open = true;
    }
    ++ex.launches;
    return ex.blas.product(x, ldx, w, ldw, out, ldo, out_dtype, M, N, K, beta, stream);
  }

  // x[M, K] . w[N, K]^T (+ bias) -> out[M, N]: the one choice of kernel per shape class
  int linear(const void* x, int x_dtype, const FmxOp& op, void* out, int out_dtype, int M) {
    const int N = op.n, K = op.k;
    const long long ldx = K, ldo = N;
    if (M == 0) return 0;
    if (x_dtype != FMX_BF16 || op.w_dtype != FMX_BF16) {
      ++ex.launches;
      return ((gemm_simple_fn)ex.k.gemm_simple)(x, op.w, op.bias, out, M, N, K, ldx, op.ldw, ldo, x_dtype, op.w_dtype,
                                                out_dtype, stream);
    }
    const bool tc_layout = bf16_operands(x, x_dtype, ldx, op.w, op.w_dtype, op.ldw, M, K);
    if (tc_layout && M <= GEMV_MAX_ROWS && (N < LIBRARY_MIN_FEATURES || op.bias != nullptr) && ex.k.gemv != nullptr) {
      ++ex.launches;
      return ((gemv_fn)ex.k.gemv)(x, ldx, op.w, op.ldw, op.bias, nullptr, 0, out, ldo, M, N, K, out_dtype, 0, 0, 0, stream);
    }
    // Products without an epilogue of this package's own run in the library from 17 rows on: with the weights
    // coming from HBM it is ahead of the one-CTA tcgen05 kernel at every size (2048 x 2048 x 8192: 47 us against 52;
    // 8192 x 4096 x 14336: 619 against 826); that kernel keeps the gate/up product, whose SiLU-mul epilogue saves a pass.
    if (op.bias != nullptr) {
      if (out_dtype != FMX_BF16) {
        ++ex.launches;
        return ((gemm_simple_fn)ex.k.gemm_simple)(x, op.w, op.bias, out, M, N, K, ldx, op.ldw, ldo, x_dtype, op.w_dtype,
                                                  out_dtype, stream);
      }
      // the bias laid under the product: both are then summed in 32-bit and rounded once
      ++ex.launches;
      if (((fill_rows_fn)ex.k.fill_rows)(op.bias, out, M, N, ldo, out_dtype, stream) != 0) return 1;
      return library_product(x, ldx, op.w, op.ldw, out, ldo, out_dtype, M, N, K, 1.0f);
    }
    return library_product(x, ldx, op.w, op.ldw, out, ldo, out_dtype, M, N, K, 0.0f);
  }

  int gate_up(const FmxOp& op) {
    const int M = rows_of(op), N = op.n, K = op.k, I = N / 2;
    const int x_dtype = ex.regs[op.in0].dtype;
    const void* x = reg(op.in0);
    void* out = reg(op.out0);
    if (M == 0) return 0;
    const bool fused = op.block > 0 && op.bias == nullptr;
    const bool tc_layout = bf16_operands(x, x_dtype, K, op.w, op.w_dtype, op.ldw, M, K);
    if (fused && tc_layout && op.block == 128 && M >= TC_MIN_ROWS && N % 256 == 0 && ex.k.gemm_tcgen05 != nullptr &&
        fills(M, N)) {
      // prompt portions: a 256-wide tile holds 128 gates and their ups, SiLU-mul in the epilogue
      ++ex.launches;
      return ((gemm_tcgen05_fn)ex.k.gemm_tcgen05)(x, K, op.w, op.ldw, out, I, nullptr, 0, M, N, K, 0, EPI_SILU_MUL, ex.sms,
                                                  d.status, stream);
    }
    if (fused && tc_layout && op.block % 16 == 0 && M <= GEMV_MAX_ROWS && ex.k.gemv != nullptr) {
      // decode steps: a block owns some gate rows and their up rows, SiLU-mul in its epilogue
      ++ex.launches;
      return ((gemv_fn)ex.k.gemv)(x, K, op.w, op.ldw, nullptr, nullptr, 0, out, I, M, N, K, FMX_BF16, op.block, 0, 0, stream);
    }
    void* both = reg(op.out1);
    if (linear(x, x_dtype, op, both, x_dtype, M) != 0) return 1;
    ++ex.launches;
    return ((silu_mul_fn)ex.k.silu_mul)(both, out, M, I, op.block > 0 ? op.block : I, x_dtype, stream);
  }

  int attention(const FmxOp& op) {
    const int g = op.group;
    const int dtype = ex.regs[op.in0].dtype;
    const long long qstride = ex.regs[op.in0].cols;
    void* qkv = reg(op.in0);
    void* out = reg(op.out0);
    const int rep = op.nh / op.nkv;
    const int* bt = g >= 0 ? d.block_tables[g] : nullptr;
    const int bt_stride = g >= 0 ? d.bt_stride[g] : 0;
    const bool tiled = dtype == FMX_BF16 && op.hd % 16 == 0 && op.hd <= 256 && qstride % 2 == 0 && op.kv != nullptr &&
                       op.fn_attn_decode != nullptr;
    const bool decode = tiled && d.all_decode && rep <= 16;
    if (!decode) {
      // rotate q (and this step's k), store k and v into the pages; then attend from the pages alone
      ++ex.launches;
      const bool store = op.store && op.kv != nullptr && g >= 0;
      if (((rope_kv_write_fn)ex.k.rope_kv_write)(qkv, d.positions, op.rot > 0 ? op.vec : nullptr,
                                                 store ? d.slot_mapping[g] : nullptr, store ? op.kv : nullptr, d.T, op.nh,
                                                 op.share_kv ? 0 : op.nkv, op.hd, op.rot, op.trad, store ? op.page_size : 1,
                                                 store ? op.num_pages : 0, qstride, dtype, d.status, stream) != 0)
        return 1;
    }
    if (decode) {
      // every row brings one token: the split kernel rotates q and the new k and stores k and v itself
      int splits = d.n_splits > 0 ? d.n_splits
                                  : ((attn_plan_fn)op.fn_attn_plan)(d.R, op.nkv, d.max_ctx_after > 1 ? d.max_ctx_after : 1, ex.sms);
      const long long need = splits <= 1 ? 0 : (long long)d.R * op.nkv * splits * 16 * (op.hd + 2);
      if (need > d.attn_scratch_floats)
        return fmx_fail("the split decode attention's workspace holds %lld floats, %lld asked for", d.attn_scratch_floats, need);
      int* tickets = need > 0 && (long long)d.R * op.nkv <= d.attn_tickets_n ? d.attn_tickets : nullptr;
      ++ex.launches;
      return ((attn_decode_fn)op.fn_attn_decode)(qkv, qstride, op.kv, bt, bt_stride, d.row_start, d.positions, out,
                                                 need > 0 ? d.attn_scratch : nullptr, need > 0 ? d.attn_scratch_floats : 0,
                                                 tickets, d.R, splits, op.nh, op.nkv, op.page_size, op.num_pages, op.scale,
                                                 op.window, d.status, op.rot > 0 ? op.vec : nullptr, op.rot, op.trad,
                                                 op.store ? 1 : 2, stream);
    }
    if (tiled) {
      // In a mixed step the decoding rows at its head go to the split decode kernel (queries rotated and keys stored
      // above) and the portions behind them to a tiled one: alone on a tile, a decoding row would walk its whole
      // context in one block.
      const int dr = rep <= 16 ? d.decode_rows : 0;
      if (dr > 0) {
        const int splits = ((attn_plan_fn)op.fn_attn_plan)(dr, op.nkv, d.decode_max_ctx > 1 ? d.decode_max_ctx : 1, ex.sms);
        const long long need = splits <= 1 ? 0 : (long long)dr * op.nkv * splits * 16 * (op.hd + 2);
        if (need > d.attn_scratch_floats)
          return fmx_fail("the split decode attention's workspace holds %lld floats, %lld asked for", d.attn_scratch_floats, need);
        int* tickets = need > 0 && (long long)dr * op.nkv <= d.attn_tickets_n ? d.attn_tickets : nullptr;
        ++ex.launches;
        if (((attn_decode_fn)op.fn_attn_decode)(qkv, qstride, op.kv, bt, bt_stride, d.row_start, d.positions, out,
                                                need > 0 ? d.attn_scratch : nullptr, need > 0 ? d.attn_scratch_floats : 0,
                                                tickets, dr, splits, op.nh, op.nkv, op.page_size, op.num_pages, op.scale,
                                                op.window, d.status, nullptr, 0, 0, 0, stream) != 0)
          return 1;
      }
      const int rows = d.R - dr, max_q = dr > 0 ? d.rest_max_q_len : d.max_q_len;
      const int* row_start = d.row_start + dr;
      const int* row_ctx = d.row_ctx + dr;
      const int* rbt = bt + (long long)dr * bt_stride;
      ++ex.launches;
      if (max_q >= TC_ATTN_MIN_TOKENS && op.tc_attention_ok && op.fn_attn_prefill_tc != nullptr && qstride % 8 == 0 &&
          aligned16(qkv))
      {
        // a grid that would leave most SMs idle shares the keys of each pair of query tiles out over several CTAs
        const int max_ctx = dr > 0 ? d.rest_max_ctx : d.max_ctx_after;
        int ks = op.fn_attn_prefill_tc_plan != nullptr && (op.hd == 64 ? 128 : 64) % op.page_size == 0
                     ? ((attn_prefill_tc_plan_fn)op.fn_attn_prefill_tc_plan)(rows, max_q, max_ctx, op.nh, op.nkv, ex.sms)
                     : 1;
        if (ks > 1 && (long long)ks * d.T * op.nh * (op.hd + 2) > d.attn_scratch_floats) ks = 1;
        if (ks > 1) ++ex.launches;
        return ((attn_prefill_tc_fn)op.fn_attn_prefill_tc)(qkv, qstride, d.T, op.kv, rbt, bt_stride, row_start, row_ctx, out,
                                                           rows, max_q, op.nh, op.nkv, op.page_size, op.num_pages,
                                                           op.scale, ks > 1 ? 2 : 0, d.status, ks, d.attn_scratch,
                                                           d.attn_scratch_floats, stream);
      }
      return ((attn_prefill_fn)op.fn_attn_prefill)(qkv, qstride, op.kv, rbt, bt_stride, row_start, row_ctx, out, rows,
                                                   max_q, op.nh, op.nkv, op.page_size, op.num_pages, op.scale,
                                                   op.window, d.status, stream);
    }
    ++ex.launches;
    return ((attention_simple_fn)ex.k.paged_attention_simple)(qkv, qstride, op.kv, bt, bt_stride, d.token_row, d.positions, out,
                                                              d.T, op.nh, op.nkv, op.hd, op.page_size, op.num_pages, op.scale,
                                                              op.window, d.R, dtype, d.status, stream);
  }

  int one(const FmxOp& op) {
    switch (op.kind) {
      case FMX_OP_EMBED: {
        const int out_dtype = ex.regs[op.out0].dtype;
        ++ex.launches;
        if (op.w_dtype == FMX_F32 && out_dtype == FMX_BF16)
          return ((gather_rows_f32_to_bf16_fn)ex.k.gather_rows_f32_to_bf16)((const float*)op.w, d.tokens, reg(op.out0), d.T,
                                                                            op.n, op.table_rows, d.status, BAD_TOKEN, stream);
        return ((gather_rows_fn)ex.k.gather_rows)(op.w, d.tokens, reg(op.out0), d.T, op.n, op.table_rows, op.w_dtype, d.status,
                                                  BAD_TOKEN, stream);
      }
      case FMX_OP_ADD_RMSNORM: {
        const int out_dtype = ex.regs[op.out0].dtype;
        const int res_dtype = op.in1 >= 0 ? ex.regs[op.in1].dtype : out_dtype;
        ++ex.launches;
        return ((add_rmsnorm_fn)ex.k.add_rmsnorm)(reg(op.in0), reg(op.in1), op.vec, reg(op.out0), rows_of(op), op.n, op.eps,
                                                  out_dtype, res_dtype, op.init, stream);
      }
      case FMX_OP_LINEAR: {
        if (op.out0 == -2 && d.greedy_ids != nullptr) {
          if (ex.k.gemv_argmax == nullptr || rows_of(op) > GEMV_MAX_ROWS)
            return fmx_fail("the greedy head takes at most %d rows of bfloat16", GEMV_MAX_ROWS);
          ++ex.launches;
          return ((gemv_argmax_fn)ex.k.gemv_argmax)(reg(op.in0), op.k, op.w, op.ldw, d.greedy_ids, d.greedy_best, d.greedy_ticket,
                                                    rows_of(op), op.n, op.k, stream);
        }
        void* out = op.out0 == -2 ? (void*)d.logits : reg(op.out0);
        return linear(reg(op.in0), ex.regs[op.in0].dtype, op, out, op.out_dtype, rows_of(op));
      }
      case FMX_OP_GATE_UP:
        return gate_up(op);
      case FMX_OP_ATTENTION:
        return attention(op);
      case FMX_OP_GATHER_ROWS:
        ++ex.launches;
        return ((gather_rows_fn)ex.k.gather_rows)(reg(op.in0), d.want, reg(op.out0), d.n_want, ex.regs[op.in0].cols, d.T,
                                                  ex.regs[op.in0].dtype, d.status, BAD_ROW, stream);
    }
    return fmx_fail("the step program holds an unknown operation %d", op.kind);
  }
};
}  // namespace

// ------------------------------------------------------------------------------------ the batch layout
namespace {
struct Layout {
  int R, Rp, T, Tp, max_blocks, max_q, max_ctx, all_decode, decode_rows, decode_max_ctx, rest_max_q, rest_max_ctx;
  long long tokens, positions, token_row, row_start, row_ctx, row_slot, want, bt[FMX_MAX_GROUPS], sm[FMX_MAX_GROUPS], total;
};

int plan_layout(const FmxBatchIn& in, Layout* L) {
  if (in.R <= 0) return fmx_fail("a step needs at least one entry");
  if (in.n_groups < 0 || in.n_groups > FMX_MAX_GROUPS) return fmx_fail("a model has at most %d cache groups here", FMX_MAX_GROUPS);
  if (in.page_size <= 0) return fmx_fail("bad page size %d", in.page_size);
  L->R = in.R;
  L->Rp = in.R > in.pad_rows ? in.R : in.pad_rows;
  long long T = 0;
  int max_blocks = in.pad_blocks > 1 ? in.pad_blocks : 1, max_q = 1, max_ctx = 1, all_decode = 1;
  for (int r = 0; r < in.R; ++r) {
    const int q = in.q_lens[r], c = in.ctx_lens[r];
    if (q <= 0 || c < 0) return fmx_fail("entry %d brings %d tokens after %d", r, q, c);
    T += q;
    const int blocks = (c + q + in.page_size - 1) / in.page_size;
    if (blocks > max_blocks) max_blocks = blocks;
    if (q > max_q) max_q = q;
    if (c + q > max_ctx) max_ctx = c + q;
    if (q != 1) all_decode = 0;
  }
  if (T + (L->Rp - L->R) > 0x7fffffffLL) return fmx_fail("too many tokens in one step");
  L->T = (int)T;
  L->Tp = (int)T + (L->Rp - L->R);
  L->max_blocks = max_blocks;
  L->max_q = max_q;
  L->max_ctx = max_ctx;
  L->all_decode = all_decode;
  // the one-token rows at the head of a mixed step
  int dr = 0;
  while (dr < in.R && in.q_lens[dr] == 1) ++dr;
  L->decode_rows = L->decode_max_ctx = L->rest_max_q = L->rest_max_ctx = 0;
  if (dr > 0 && dr < in.R) {
    L->decode_rows = dr;
    for (int r = 0; r < dr; ++r)
      if (in.ctx_lens[r] + 1 > L->decode_max_ctx) L->decode_max_ctx = in.ctx_lens[r] + 1;
    for (int r = dr; r < in.R; ++r) {
      if (in.q_lens[r] > L->rest_max_q) L->rest_max_q = in.q_lens[r];
      if (in.ctx_lens[r] + in.q_lens[r] > L->rest_max_ctx) L->rest_max_ctx = in.ctx_lens[r] + in.q_lens[r];
    }
  }
  long long at = 0;
  auto take = [&](long long n) { at = (at + 3) / 4 * 4; const long long o = at; at += n; return o; };   // 16-byte starts
  L->tokens = take(L->Tp);
  L->positions = take(L->Tp);
  L->token_row = take(L->Tp);
  L->row_start = take(L->Rp + 1);
  L->row_ctx = take(L->Rp);
  L->row_slot = take(L->Rp);
  L->want = take(in.n_want);
  for (int g = 0; g < in.n_groups; ++g) {
    L->bt[g] = take((long long)L->Rp * max_blocks);
    L->sm[g] = take(2LL * L->Tp);                        // 64-bit entries
  }
  L->total = (at + 3) / 4 * 4;
  return 0;
}
}  // namespace

FMX_EXPORT long long fmx_exec_layout_ints(const FmxBatchIn* in) {
  Layout L;
  if (plan_layout(*in, &L) != 0) return -1;
  return L.total;
}

FMX_EXPORT int fmx_exec_layout(const FmxBatchIn* in, int* host, int* dev, long long capacity_ints, FmxStepDesc* desc,
                               cudaStream_t stream) {
  Layout L;
  if (plan_layout(*in, &L) != 0) return 1;
  if (L.total > capacity_ints)
    return fmx_fail("the step's description takes %lld ints, the buffers hold %lld", L.total, capacity_ints);
  const int ps = in->page_size;
  int* tok = host + L.tokens;
  int* pos = host + L.positions;
  int* trow = host + L.token_row;
  int* rstart = host + L.row_start;
  int* rctx = host + L.row_ctx;
  int* rslot = host + L.row_slot;
  int off = 0;
  for (int r = 0; r < L.R; ++r) {
    const int q = in->q_lens[r], c = in->ctx_lens[r];
    memcpy(tok + off, in->tokens + off, (size_t)q * sizeof(int));
    for (int i = 0; i < q; ++i) {
      pos[off + i] = c + i;
      trow[off + i] = r;
    }
    rstart[r] = off;
    rctx[r] = c;
    rslot[r] = in->slots[r];
    off += q;
  }
  for (int r = L.R; r < L.Rp; ++r) {                     // padding rows: one token, no context, stored nowhere, no slot
    tok[off] = 0;
    pos[off] = -1;
    trow[off] = r;
    rstart[r] = off;
    rctx[r] = 0;
    rslot[r] = -1;
    ++off;
  }
  rstart[L.Rp] = off;
  for (int i = 0; i < in->n_want; ++i) {
    if (in->want[i] < 0 || in->want[i] >= L.Tp) return fmx_fail("wanted place %d lies outside the step's %d tokens", in->want[i], L.Tp);
    host[L.want + i] = in->want[i];
  }
  for (int g = 0; g < in->n_groups; ++g) {
    int* bt = host + L.bt[g];
    long long* sm = reinterpret_cast<long long*>(host + L.sm[g]);
    const int cols = in->mirror_cols[g] < L.max_blocks ? in->mirror_cols[g] : L.max_blocks;
    for (long long i = 0; i < (long long)L.Rp * L.max_blocks; ++i) bt[i] = -1;
    int t = 0;
    for (int r = 0; r < L.R; ++r) {
      const int q = in->q_lens[r], c = in->ctx_lens[r];
      int* row = bt + (long long)r * L.max_blocks;
      memcpy(row, in->mirror[g] + (long long)in->slots[r] * in->mirror_cols[g], (size_t)cols * sizeof(int));
      for (int i = 0; i < q; ++i, ++t) {
        const int p = c + i, b = p / ps;
        const int page = b < L.max_blocks ? row[b] : -1;
        sm[t] = page < 0 ? -1 : (long long)page * ps + p % ps;
      }
    }
    for (; t < L.Tp; ++t) sm[t] = -1;
  }
  if (dev == nullptr) {
    dev = host;                                          // no device: the description's pointers then point into `host`
  } else {
    cudaError_t e = cudaMemcpyAsync(dev, host, (size_t)L.total * sizeof(int), cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) return fmx_fail("copying the step's description to the device: %s", cudaGetErrorString(e));
  }
  desc->T = L.Tp;
  desc->R = L.Rp;
  desc->n_want = in->n_want;
  desc->max_q_len = L.max_q;
  desc->max_ctx_after = L.max_ctx;
  desc->all_decode = L.all_decode;
  desc->decode_rows = L.decode_rows;
  desc->decode_max_ctx = L.decode_max_ctx;
  desc->rest_max_q_len = L.rest_max_q;
  desc->rest_max_ctx = L.rest_max_ctx;
  desc->n_splits = 0;
  desc->n_groups = in->n_groups;
  desc->tokens = dev + L.tokens;
  desc->positions = dev + L.positions;
  desc->token_row = dev + L.token_row;
  desc->row_start = dev + L.row_start;
  desc->row_ctx = dev + L.row_ctx;
  desc->row_slot = dev + L.row_slot;
  desc->want = dev + L.want;
  for (int g = 0; g < in->n_groups; ++g) {
    desc->block_tables[g] = dev + L.bt[g];
    desc->bt_stride[g] = L.max_blocks;
    desc->slot_mapping[g] = reinterpret_cast<const long long*>(dev + L.sm[g]);
  }
  return 0;
}

// ------------------------------------------------------------------------------------ the executor
FMX_EXPORT void* fmx_exec_create(const FmxOp* ops, int n_ops, const FmxReg* regs, int n_regs,
                                 const FmxKernelTable* kernels, int sms, const char* cublas_path, void* cublas_workspace,
                                 long long cublas_workspace_bytes) {
  if (ops == nullptr || regs == nullptr || kernels == nullptr || n_ops <= 0 || n_regs <= 0) {
    fmx_fail("fmx_exec_create: an empty program");
    return nullptr;
  }
  if (kernels->gather_rows == nullptr || kernels->add_rmsnorm == nullptr || kernels->gemm_simple == nullptr ||
      kernels->rope_kv_write == nullptr || kernels->paged_attention_simple == nullptr || kernels->silu_mul == nullptr ||
      kernels->fill_rows == nullptr || kernels->gather_rows_f32_to_bf16 == nullptr) {
    fmx_fail("fmx_exec_create: the common kernel library's entry points are missing");
    return nullptr;
  }
  for (int i = 0; i < n_ops; ++i) {
    const FmxOp& op = ops[i];
    const int refs[4] = {op.in0, op.in1, op.out0, op.out1};
    for (int r : refs)
      if (r >= n_regs || r < -2) {
        fmx_fail("fmx_exec_create: operation %d names register %d of %d", i, r, n_regs);
        return nullptr;
      }
    if (op.kind == FMX_OP_ATTENTION && (op.nh <= 0 || op.nkv <= 0 || op.nh % op.nkv || op.group >= FMX_MAX_GROUPS)) {
      fmx_fail("fmx_exec_create: operation %d has bad attention sizes", i);
      return nullptr;
    }
  }
  Executor* ex = new Executor();
  ex->ops.assign(ops, ops + n_ops);
  ex->regs.assign(regs, regs + n_regs);
  ex->k = *kernels;
  ex->sms = sms > 0 ? sms : fmx_num_sms();
  if (cublas_path != nullptr) {
    ex->blas_path_store.assign(cublas_path, cublas_path + strlen(cublas_path) + 1);
    ex->blas_path = ex->blas_path_store.data();
  }
  ex->blas_ws = cublas_workspace;
  ex->blas_ws_bytes = cublas_workspace_bytes;
  return ex;
}

FMX_EXPORT void fmx_exec_destroy(void* exec) {
  Executor* ex = static_cast<Executor*>(exec);
  if (ex == nullptr) return;
  ex->blas.close();
  delete ex;
}

FMX_EXPORT long long fmx_exec_arena_bytes(void* exec, int T) {
  return place_registers(*static_cast<Executor*>(exec), T, nullptr);
}

// Sizes of the structures shared with the loader, which checks its mirrors against them.
FMX_EXPORT void fmx_exec_struct_sizes(int* sizes) {
  sizes[0] = (int)sizeof(FmxOp);
  sizes[1] = (int)sizeof(FmxStepDesc);
  sizes[2] = (int)sizeof(FmxBatchIn);
  sizes[3] = (int)sizeof(FmxKernelTable);
  sizes[4] = (int)sizeof(FmxReg);
}

FMX_EXPORT long long fmx_exec_launches(void* exec) { return static_cast<Executor*>(exec)->launches; }

FMX_EXPORT int fmx_exec_forward(void* exec, const FmxStepDesc* desc, cudaStream_t stream) {
  Executor* ex = static_cast<Executor*>(exec);
  if (ex == nullptr || desc == nullptr) return fmx_fail("fmx_exec_forward: no executor or no step");
  if (desc->T <= 0 || desc->R <= 0) return fmx_fail("fmx_exec_forward: an empty step");
  const long long need = place_registers(*ex, desc->T, &ex->offsets);
  if (desc->arena == nullptr || need > desc->arena_bytes)
    return fmx_fail("fmx_exec_forward: a step of %d tokens needs %lld bytes of arena, %lld given", desc->T, need, desc->arena_bytes);
  if (((uintptr_t)desc->arena & 255) != 0) return fmx_fail("fmx_exec_forward: the arena must start on a 256-byte boundary");
  Run run{*ex, *desc, stream};
  for (const FmxOp& op : ex->ops) {
    if (op.wanted_rows && desc->n_want == 0) continue;      // nothing is wanted: the tail of the program has no rows
    if (run.one(op) != 0) return 1;
  }
  return 0;
}
