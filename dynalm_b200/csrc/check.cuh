// The checked build of the kernels (-DDL_CHECK, DYNALM_CHECK=1 in the environment of the Python package).
//
// A kernel takes some of its indices from device memory: token ids, the rows a norm gathers, the request of a
// row, the pages of a block table, the query tiles of the prompt attention, the places that decoded tokens are
// fed back from. The host fills all of them and checks them before a step, so a wrong one means a fault of the
// host code; without a memory checker it would show as a silent wrong read or a fault of the whole context.
// In a checked build every such index is compared with its range before it is used. A violation is written to a
// record in device memory (the first one wins: code, value, range, block and thread), the access is not made
// (a store is skipped; a load goes to element 0 of the same array, whose result the kernel then uses as it
// would have used the wrong one), and nothing traps, so the context stays usable. The host reads the record
// with dl_check_take after the launch and raises an error that says which index was wrong.
//
// The ranges that a kernel does not get as arguments (pages of the cache, rows of the block table, rows of the
// step, the vocabulary) are set by the host with dl_check_limits, in stream order before the launch; a limit of
// 0 means "not known" and is not checked. Every kernel library carries its own record and limits.
//
// Without -DDL_CHECK the helpers below are the plain loads and cost nothing. This is the stand-in for the
// reference's sanitizer builds (cmake/EngineCompilerFlags.cmake:26-56) on a machine without a memory checker.
#pragma once

#define DL_CK_TOKEN 1     // a token id outside the vocabulary
#define DL_CK_ROW 2       // a gathered row outside the rows of the step
#define DL_CK_REQUEST 3   // a row's request outside the block table
#define DL_CK_BLOCK 4     // a position whose block lies outside the request's row of the block table
#define DL_CK_PAGE 5      // a page id outside the pool (-1: a page that a window has given back)
#define DL_CK_PLACE 6     // a place in the chosen ids outside the array
#define DL_CK_TILE 7      // a query tile whose rows lie outside the step
#define DL_CK_PART 8      // a part of a query tile outside its parts, or its records outside the scratch

namespace dl {

#ifdef DL_CHECK

struct CheckLimits {
  int pages, requests, rows, vocab;
};
static __device__ CheckLimits g_limits;
static __device__ long long g_check[8];     // code, value, lo, hi, blockIdx.x, blockIdx.y, blockIdx.z, threadIdx.x

__device__ __noinline__ bool check_failed(int code, long long v, long long lo, long long hi) {
  if (atomicCAS(reinterpret_cast<unsigned long long*>(&g_check[0]), 0ull, static_cast<unsigned long long>(code)) == 0ull) {
    g_check[1] = v;
    g_check[2] = lo;
    g_check[3] = hi;
    g_check[4] = blockIdx.x;
    g_check[5] = blockIdx.y;
    g_check[6] = blockIdx.z;
    g_check[7] = threadIdx.x;
  }
  return false;
}

// v in [lo, hi), or a record of the violation; a range with hi <= lo is not known and passes.
__device__ __forceinline__ bool check_range(int code, long long v, long long lo, long long hi) {
  return hi <= lo || (v >= lo && v < hi) || check_failed(code, v, lo, hi);
}

__device__ __forceinline__ int ck_token(int id, int vocab) { return check_range(DL_CK_TOKEN, id, 0, vocab) ? id : 0; }
__device__ __forceinline__ int ck_row(int r, int rows) { return check_range(DL_CK_ROW, r, 0, rows) ? r : 0; }
__device__ __forceinline__ int ck_row(int r) { return ck_row(r, g_limits.rows); }
__device__ __forceinline__ int ck_request(int req) { return check_range(DL_CK_REQUEST, req, 0, g_limits.requests) ? req : 0; }
__device__ __forceinline__ int ck_place(int p, int n) { return check_range(DL_CK_PLACE, p, 0, n) ? p : 0; }
// the page of block `block` of a request's table row, for a load: page 0 after a violation
__device__ __forceinline__ int ck_page(const int* table, int block, int max_blocks) {
  if (!check_range(DL_CK_BLOCK, block, 0, max_blocks)) return 0;
  const int page = table[block];
  return check_range(DL_CK_PAGE, page, 0, g_limits.pages) ? page : 0;
}
// the same for a store: -1 after a violation, and the caller skips the store
__device__ __forceinline__ int ck_page_store(const int* table, int block, int max_blocks) {
  if (!check_range(DL_CK_BLOCK, block, 0, max_blocks)) return -1;
  const int page = table[block];
  return check_range(DL_CK_PAGE, page, 0, g_limits.pages) ? page : -1;
}
// a query tile (request, first row, rows, first position): rows inside the step, request inside the table;
// after a violation a tile of no rows
__device__ __forceinline__ int4 ck_tile(int4 t) {
  const bool ok = check_range(DL_CK_REQUEST, t.x, 0, g_limits.requests) &&
                  check_range(DL_CK_TILE, t.y, 0, g_limits.rows) &&
                  check_range(DL_CK_TILE, static_cast<long long>(t.y) + t.z, 0, static_cast<long long>(g_limits.rows) + 1) &&
                  check_range(DL_CK_TILE, t.z, 0, 1 << 30) && check_range(DL_CK_BLOCK, t.w, 0, 1 << 30);
  return ok ? t : make_int4(0, 0, 0, 0);
}

// a word that names one part of a query tile whose keys are dealt over blocks (part | parts << 8 | first record << 16):
// the part among its parts, its records among the `records` of scratch; after a violation 0 (a whole tile), so that
// nothing is written to scratch
__device__ __forceinline__ int ck_part_word(int word, int records) {
  const int part = word & 0xff, parts = (word >> 8) & 0xff, first = word >> 16;
  if (parts <= 1) return word;
  const bool ok = check_range(DL_CK_PART, part, 0, parts) && check_range(DL_CK_PART, static_cast<long long>(first) + parts, 0,
                                                                        static_cast<long long>(records) + 1);
  return ok ? word : 0;
}

#else

__device__ __forceinline__ int ck_part_word(int word, int) { return word; }
__device__ __forceinline__ int ck_token(int id, int) { return id; }
__device__ __forceinline__ int ck_row(int r, int) { return r; }
__device__ __forceinline__ int ck_row(int r) { return r; }
__device__ __forceinline__ int ck_request(int req) { return req; }
__device__ __forceinline__ int ck_place(int p, int) { return p; }
__device__ __forceinline__ int ck_page(const int* table, int block, int) { return table[block]; }
__device__ __forceinline__ int ck_page_store(const int* table, int block, int) { return table[block]; }
__device__ __forceinline__ int4 ck_tile(int4 t) { return t; }

#endif

}  // namespace dl

#ifdef DL_CHECK
// Sets the ranges the kernels of this library check against, in stream order (0: not known).
DL_EXPORT int dl_check_limits(int pages, int requests, int rows, int vocab, cudaStream_t stream) {
  const dl::CheckLimits l = {pages, requests, rows, vocab};
  return static_cast<int>(cudaMemcpyToSymbolAsync(dl::g_limits, &l, sizeof(l), 0, cudaMemcpyHostToDevice, stream));
}

// Waits for the stream, copies this library's record of the first violation into out[8] and clears it.
// out[0] == 0: none.
DL_EXPORT int dl_check_take(long long* out, cudaStream_t stream) {
  cudaError_t e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemcpyFromSymbol(out, dl::g_check, 8 * sizeof(long long));
  if (e != cudaSuccess) return static_cast<int>(e);
  if (out[0] != 0) {
    const long long zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    e = cudaMemcpyToSymbol(dl::g_check, zero, sizeof(zero));
  }
  return static_cast<int>(e);
}
#endif
