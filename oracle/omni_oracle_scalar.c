/* Scalar CPU restatement of the reference's correctness-first kernel.  TEST INFRASTRUCTURE ONLY.
 *
 * Follows the per-row loop of omni-attn-mma/mma/attn_naive.cu:95-301: one output row at a time,
 * walk the row's listed KV blocks, pass 1 finds the maximum scaled score over the allowed keys,
 * pass 2 accumulates exp(score - max) and exp(score - max) * V, then normalises; a row with no
 * allowed key yields zeros (attn_naive.cu:178-183). Block semantics as in that kernel:
 *   MASKED skipped (:109); keys clipped to seqlen_orig (:113); CAUSAL keeps key <= query by absolute
 *   position (:135-141); PARTIAL looks the element up in the byte mask pool (:143-155).
 * One deliberate switch: a PARTIAL entry with no usable pool index is skipped by that kernel
 * (:120-131) but expanded as CAUSAL by the torch path (omni-attn-mma/omni_attn_torch.py:140-143);
 * `partial_fallback_causal` selects which of the two is computed.
 * Rows are independent, so the caller passes the list of (batch*head, query) rows it wants; that is
 * how full-size configurations are spot-checked without an N x N score matrix. Dot products are
 * accumulated in float as the kernel does, the row sums in double. It also returns the
 * log-sum-exp of each row (not in the reference; needed to check the LSE output).
 *
 * Build: gcc -O3 -fopenmp -shared -fPIC omni_oracle_scalar.c -o libomni_oracle_scalar.so -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

enum { T_MASKED = 0, T_CAUSAL = 1, T_FULL = 2, T_PARTIAL = 3 };

static float dotf(const float* a, const float* b, int d) {
  float s = 0.f;
  for (int i = 0; i < d; ++i) s += a[i] * b[i];
  return s;
}

int omni_oracle_rows(const float* q, const float* k, const float* v, const int32_t* kv_num_blocks,
                     const int32_t* kv_indices, const int32_t* block_mask_types,
                     const int32_t* partial_idx, const uint8_t* partial_masks, int num_partial, int BH,
                     int N, int seqlen_orig, int D, int block, int max_blocks, float scale,
                     const int32_t* rows_bh, const int32_t* rows_q, int n_rows, float* out, float* lse,
                     int partial_fallback_causal) {
  const int nq = (N + block - 1) / block;
  int bad = 0;
#pragma omp parallel for schedule(dynamic, 8)
  for (int r = 0; r < n_rows; ++r) {
    const int bh = rows_bh[r];
    const int qi = rows_q[r];
    float* o = out + (size_t)r * D;
    for (int d = 0; d < D; ++d) o[d] = 0.f;
    lse[r] = -INFINITY;
    if (bh < 0 || bh >= BH || qi < 0 || qi >= N) {
      bad = 1;
      continue;
    }
    if (qi >= seqlen_orig) continue; /* padding row: zeros (attn_naive.cu:65-72) */
    const int qb = qi / block;
    const size_t head = (size_t)bh * N * D;
    const float* qrow = q + head + (size_t)qi * D;
    const size_t lbase = ((size_t)bh * nq + qb) * max_blocks;
    int nlist = kv_num_blocks[(size_t)bh * nq + qb];
    if (nlist > max_blocks) nlist = max_blocks;
    double* acc = (double*)calloc((size_t)D, sizeof(double));
    float mx = -INFINITY;
    double sum = 0.0;
    for (int pass = 0; pass < 2; ++pass) {
      for (int i = 0; i < nlist; ++i) {
        const int kb = kv_indices[lbase + i];
        int t = block_mask_types[lbase + i];
        if (t == T_MASKED || t < 0 || t > 3) continue;
        if (kb < 0 || kb >= nq) continue;
        const int k0 = kb * block;
        int k1 = k0 + block;
        if (k1 > seqlen_orig) k1 = seqlen_orig;
        int pi = -1;
        if (t == T_PARTIAL) {
          if (partial_idx != NULL && partial_masks != NULL) pi = partial_idx[lbase + i];
          if (pi < 0 || pi >= num_partial) {
            if (!partial_fallback_causal) continue;
            t = T_CAUSAL;
          }
        }
        if (t == T_CAUSAL) {
          if (qi < k0) continue;
          if (k1 > qi + 1) k1 = qi + 1;
        }
        for (int kj = k0; kj < k1; ++kj) {
          if (t == T_PARTIAL) {
            const size_t off = ((size_t)pi * block + (size_t)(qi - qb * block)) * block + (size_t)(kj - k0);
            if (!partial_masks[off]) continue;
          }
          const float s = dotf(qrow, k + head + (size_t)kj * D, D) * scale;
          if (pass == 0) {
            if (s > mx) mx = s;
          } else {
            const float w = expf(s - mx);
            sum += w;
            const float* vrow = v + head + (size_t)kj * D;
            for (int d = 0; d < D; ++d) acc[d] += (double)w * vrow[d];
          }
        }
      }
      if (pass == 0 && mx == -INFINITY) break; /* nothing attended: zeros */
    }
    if (sum > 0.0) {
      for (int d = 0; d < D; ++d) o[d] = (float)(acc[d] / sum);
      lse[r] = mx + (float)log(sum);
    }
    free(acc);
  }
  return bad ? -1 : 0;
}
