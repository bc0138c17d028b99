// The device's copy of the block tables, brought up to date.
//
// The device keeps one table row per request slot and cache group: tables[group][slot][block] = page. A step
// sends only the entries that have changed since the step before (new pages at the end of a growing request,
// pages a window has given back, copies made before a write into a shared page) as (group, slot, block, page)
// quadruples, and this kernel writes them in. Entries outside the tables are skipped (a checked build records
// them). The reference uploads each sequence's whole table with every forward pass
// (dynalm/src/model/transformer.cpp:635-636); at its context lengths that is small.
#include "common.cuh"

namespace dl {

__global__ void table_update_kernel(int* __restrict__ tables, const int4* __restrict__ updates, int n, int groups,
                                    int slots, int max_blocks) {
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int4 u = updates[i];
#ifdef DL_CHECK
  if (!check_range(DL_CK_REQUEST, u.y, 0, slots) || !check_range(DL_CK_BLOCK, u.z, 0, max_blocks)) return;
#endif
  if (u.x < 0 || u.x >= groups || u.y < 0 || u.y >= slots || u.z < 0 || u.z >= max_blocks) return;
  tables[(static_cast<size_t>(u.x) * slots + u.y) * max_blocks + u.z] = u.w;
}

// Pages that were just handed out are cleared in every array of their cache group: storage [planes][pages][page_bytes],
// fresh = pairs (group id, page); one block per (pair, plane), pairs of another group are skipped.
__global__ void zero_pages_kernel(unsigned char* __restrict__ storage, long long page_bytes, long long plane_bytes,
                                  const int2* __restrict__ fresh, int group, int pages) {
  pdl_wait();
  pdl_trigger();
  const int2 what = fresh[blockIdx.x];
  if (what.x != group || what.y < 0 || what.y >= pages) return;
  unsigned char* p = storage + static_cast<long long>(blockIdx.y) * plane_bytes + static_cast<long long>(what.y) * page_bytes;
  const long long vecs = page_bytes / 16;
  uint4* v = reinterpret_cast<uint4*>(p);
  for (long long i = threadIdx.x; i < vecs; i += blockDim.x) v[i] = make_uint4(0, 0, 0, 0);
  for (long long i = vecs * 16 + threadIdx.x; i < page_bytes; i += blockDim.x) p[i] = 0;
}

}  // namespace dl

// storage: a cache group's arrays, `planes` arrays of `pages` pages of page_bytes bytes each (16-byte aligned pages);
// fresh: int32 [n, 2] = (group id, page), 8-byte aligned. Pages of `group` are set to zero in every plane.
DL_EXPORT int dl_zero_pages(void* storage, long long page_bytes, int pages, int planes, const void* fresh, int n, int group,
                            cudaStream_t stream) {
  if (n <= 0 || planes <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(fresh) & 7) || (reinterpret_cast<uintptr_t>(storage) & 15) || (page_bytes & 15) || planes > 65535)
    return DL_ERR_UNSUPPORTED;
  return dl::launch(dl::zero_pages_kernel, dim3(n, planes), dim3(256), 0, stream, static_cast<unsigned char*>(storage),
                    page_bytes, page_bytes * pages, static_cast<const int2*>(fresh), group, pages);
}

// tables: int32 [groups, slots, max_blocks]; updates: int32 [n, 4] = (group, slot, block, page), 16-byte aligned.
DL_EXPORT int dl_table_updates(int* tables, const void* updates, int n, int groups, int slots, int max_blocks,
                               cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(updates) & 15) != 0) return DL_ERR_UNSUPPORTED;
  return dl::launch(dl::table_update_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, tables,
                    static_cast<const int4*>(updates), n, groups, slots, max_blocks);
}
