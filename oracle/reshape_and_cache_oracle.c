/*
 * CPU oracle for reshape_and_cache, plain C.  TEST INFRASTRUCTURE ONLY: it is loaded by the
 * tests (and may be timed as the CPU baseline); the product never links or calls it.
 *
 * Restates the index arithmetic of the reference kernel
 * (csrc/opdev/op_kernel/reshape_and_cache_ex.cpp:47-69) and of its golden
 * (benchmark/test_reshape_and_cache.py:6-25) on 16-bit payloads:
 *   NZ  cache [pages, C, P, 16]:  cache[s/P][c][s%P][j] = flat(key[t])[c*16 + j]
 *   NHD cache [pages, P, Hkv, D]: cache[s/P][s%P][h][d] = key[t][h][d]
 * Tokens are visited in order, so a repeated slot keeps the later token, as in the
 * reference's sequential loop.  Slots outside [0, pages*P) are skipped (:50).
 * Pinned by tests/test_oracle.py against fixtures made with the reference's own golden.
 */
#include <stdint.h>
#include <string.h>

void oracle_reshape_and_cache(const uint16_t* key, const uint16_t* value, uint16_t* key_cache,
                              uint16_t* value_cache, const int32_t* slots, int64_t num_tokens,
                              int64_t row_elems, int64_t pages, int64_t chunks, int64_t page_size,
                              int layout_nhd) {
  const int with_value = value != 0 && value_cache != 0;
  for (int64_t t = 0; t < num_tokens; ++t) {
    const int64_t s = slots[t];
    if (s < 0 || s >= pages * page_size) continue;
    const uint16_t* k = key + t * row_elems;
    const uint16_t* v = with_value ? value + t * row_elems : 0;
    if (layout_nhd) {
      memcpy(key_cache + s * row_elems, k, (size_t)row_elems * 2);
      if (with_value) memcpy(value_cache + s * row_elems, v, (size_t)row_elems * 2);
      continue;
    }
    const int64_t page = s / page_size, off = s % page_size;
    for (int64_t c = 0; c < chunks; ++c) {
      for (int j = 0; j < 16; ++j) {
        const int64_t e = c * 16 + j;
        if (e >= row_elems) break;
        const int64_t dst = ((page * chunks + c) * page_size + off) * 16 + j;
        key_cache[dst] = k[e];
        if (with_value) value_cache[dst] = v[e];
      }
    }
  }
}
