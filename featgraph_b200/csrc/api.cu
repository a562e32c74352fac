// Error reporting, version and the host-only partitioning helpers of the C ABI.
#include <algorithm>

#include "common.cuh"

namespace fg {

std::string& last_error() {
  static thread_local std::string msg;
  return msg;
}

int fail(int code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  last_error() = buf;
  return code;
}

static thread_local LaunchOptions g_next_options;

LaunchOptions take_launch_options() {
  const LaunchOptions o = g_next_options;
  g_next_options = LaunchOptions();
  return o;
}

}  // namespace fg

extern "C" int fg_next_launch_options(int32_t flags, int32_t max_ctas) {
  const int32_t known = FG_LAUNCH_PROGRAMMATIC | FG_SPMM_GIANT_ROWS_ONLY |
                        FG_SPMM_SKIP_GIANT_ROWS | FG_SDDMM_TMA_STAGING | FG_SPMM_LONG_ROWS_ONLY |
                        FG_SPMM_SKIP_LONG_ROWS | FG_SDDMM_ROW_REGISTERS;
  const int32_t cuts = flags & (FG_SPMM_GIANT_ROWS_ONLY | FG_SPMM_SKIP_GIANT_ROWS |
                                FG_SPMM_LONG_ROWS_ONLY | FG_SPMM_SKIP_LONG_ROWS);
  if ((flags & ~known) != 0 || max_ctas < 0 || (cuts & (cuts - 1)) != 0)  // at most one cut
    return fg::fail(FG_ERR_INVALID_ARGUMENT, "bad launch options: flags=%d max_ctas=%d", (int)flags,
                    (int)max_ctas);
  fg::g_next_options.flags = flags;
  fg::g_next_options.max_ctas = max_ctas;
  return FG_OK;
}

extern "C" const char* fg_last_error_string(void) { return fg::last_error().c_str(); }

extern "C" const char* fg_version(void) { return "0.1.0"; }

extern "C" int fg_shard_rows_by_nnz(const int32_t* indptr, int64_t n_rows, int32_t world,
                                    int64_t* bounds) {
  using namespace fg;
  if (!indptr || !bounds) return fail(FG_ERR_INVALID_ARGUMENT, "null indptr or bounds");
  if (n_rows < 0 || world <= 0)
    return fail(FG_ERR_INVALID_ARGUMENT, "bad n_rows=%lld or world=%d", (long long)n_rows,
                (int)world);
  for (int64_t r = 0; r < n_rows; ++r)
    if (indptr[r + 1] < indptr[r])
      return fail(FG_ERR_INVALID_ARGUMENT, "indptr decreases at row %lld", (long long)r);
  const int64_t nnz = n_rows > 0 ? (int64_t)indptr[n_rows] - indptr[0] : 0;
  bounds[0] = 0;
  for (int32_t k = 1; k < world; ++k) {
    // First row boundary whose prefix count reaches k/world of the nonzeros,
    // or the nearer of its two neighbours; never below the previous bound.
    const int64_t target = indptr[0] + (nnz * k) / world;
    const int32_t* it = std::lower_bound(indptr, indptr + n_rows + 1, (int32_t)target);
    int64_t b = it - indptr;
    if (b > 0 && b <= n_rows &&
        (target - indptr[b - 1]) < ((int64_t)indptr[std::min(b, n_rows)] - target))
      b = b - 1;
    b = std::min<int64_t>(std::max<int64_t>(b, bounds[k - 1]), n_rows);
    bounds[k] = b;
  }
  bounds[world] = n_rows;
  return FG_OK;
}

extern "C" int fg_shard_edges(int64_t nnz, int32_t world, int64_t* bounds) {
  using namespace fg;
  if (!bounds) return fail(FG_ERR_INVALID_ARGUMENT, "null bounds");
  if (nnz < 0 || world <= 0)
    return fail(FG_ERR_INVALID_ARGUMENT, "bad nnz=%lld or world=%d", (long long)nnz, (int)world);
  const int64_t chunk = ((nnz + world - 1) / world + 31) / 32 * 32;
  for (int32_t k = 0; k <= world; ++k) bounds[k] = std::min<int64_t>(nnz, chunk * k);
  return FG_OK;
}
