// Host-side reader for the reference's dataset text layout.
//
// The reference's read_data (include/mcmc/io.h:42-80 there) scans a
// whitespace-separated table with fscanf: TOTAL_COLS header tokens are thrown
// away, then every row has TOTAL_COLS tokens of which the first SKIP_COLS are
// ignored, the next one is the label, the next 22 are the features and the rest
// is ignored (global_params.h:61-65).  This reader takes the same layout with
// the sizes as arguments, parses the file in one pass over a memory image
// (strtof per kept token, no per-token stdio call) and applies the feature
// scaling the reference does in a separate device pass (main.h:162-164).
#include <errno.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string>
#include <vector>

#include "../../include/mcmc_b200.h"

// defined in api.cu: the library-wide last-error text
void mcmc_b200_set_last_error(const std::string& msg);

#define API extern "C" __attribute__((visibility("default")))

namespace {
int io_fail(const std::string& msg) {
  mcmc_b200_set_last_error(msg);
  return MCMC_B200_ERR_INVALID;
}
inline bool is_space(char c) { return c == ' ' || c == '\t' || c == '\n' || c == '\r' || c == '\f' || c == '\v'; }
}  // namespace

API int mcmc_b200_read_table(const char* path, int64_t rows, int total_cols, int skip_cols, int D,
                             float feature_scale, float* x_out, float* y_out) {
  if (!path || rows < 0 || total_cols < 1 || skip_cols < 0 || D < 1 || skip_cols + 1 + D > total_cols ||
      !x_out || !y_out)
    return io_fail("bad arguments");
  FILE* fp = fopen(path, "rb");
  if (!fp) return io_fail(std::string("cannot open '") + path + "'");
  std::vector<char> buf;
  {
    fseek(fp, 0, SEEK_END);
    const long sz = ftell(fp);
    fseek(fp, 0, SEEK_SET);
    if (sz < 0) { fclose(fp); return io_fail("cannot size the file"); }
    buf.resize((size_t)sz + 1);
    const size_t got = fread(buf.data(), 1, (size_t)sz, fp);
    fclose(fp);
    buf[got] = '\0';
    buf.resize(got + 1);
  }
  const char* p = buf.data();
  const char* end = buf.data() + buf.size() - 1;
  auto skip_token = [&]() -> bool {
    while (p < end && is_space(*p)) ++p;
    if (p >= end) return false;
    while (p < end && !is_space(*p)) ++p;
    return true;
  };
  auto read_float = [&](float& v) -> bool {
    while (p < end && is_space(*p)) ++p;
    if (p >= end) return false;
    char* q = nullptr;
    errno = 0;
    v = strtof(p, &q);
    if (q == p) return false;
    p = q;
    return true;
  };
  for (int j = 0; j < total_cols; ++j)
    if (!skip_token()) return io_fail("file ends inside the header");
  const int label_col = skip_cols, first_feat = skip_cols + 1, last_feat = skip_cols + D;
  for (int64_t i = 0; i < rows; ++i) {
    for (int j = 0; j < total_cols; ++j) {
      bool ok;
      if (j == label_col) {
        ok = read_float(y_out[i]);
      } else if (j >= first_feat && j <= last_feat) {
        float v = 0.f;
        ok = read_float(v);
        x_out[i * D + (j - first_feat)] = v * feature_scale;
      } else {
        ok = skip_token();
      }
      if (!ok) {
        char msg[160];
        snprintf(msg, sizeof msg, "file ends or has a non-numeric field at row %lld, column %d", (long long)i, j);
        return io_fail(msg);
      }
    }
  }
  return MCMC_B200_OK;
}
