/* TEST INFRASTRUCTURE ONLY (checker side).
 *
 * Plain-C restatement of the reference's message-passing operators, written to
 * reproduce the reference CPU bodies' arithmetic ORDER (so fp32 results are
 * bit-identical to them) while being independent code.  Citations are to files
 * of the reference project (jittor_geometric/...).  Only tests, the smoke check
 * and the benchmark's CPU-baseline leg may load this library; the product path
 * never does.
 *
 * Conventions: indices int32, values fp32, dense matrices row-major,
 * `off` has n+1 entries, segment v = [off[v], off[v+1]).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* Stable counting sort of a COO list by `key` (ops/cpp/cootocsr_op.cc:35-53 with
 * key = source; ops/cpp/cootocsc_op.cc:33-51 with key = destination).  Entry i
 * lands at off[key[i]] + #{j < i : key[j] == key[i]}. */
void orc_coo_compress(const int32_t* key, const int32_t* other, const float* w, int64_t E,
                      int32_t n, int32_t* off, int32_t* idx, float* out_w) {
    memset(off, 0, sizeof(int32_t) * ((size_t)n + 1));
    for (int64_t i = 0; i < E; i++) off[key[i] + 1]++;
    for (int32_t v = 0; v < n; v++) off[v + 1] += off[v];
    int32_t* fill = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n > 0 ? n : 1));
    memcpy(fill, off, sizeof(int32_t) * (size_t)n);
    for (int64_t i = 0; i < E; i++) {
        int32_t p = fill[key[i]]++;
        idx[p] = other[i];
        out_w[p] = w[i];
    }
    free(fill);
}

/* Weighted segment aggregation (ops/cpp/aggregate_op.cc:42-58 AVX branch and
 * :61-69 scalar branch): out[v,:] = sum_{j in seg(v)} x[idx[j],:] * w[j], terms
 * added in ascending j, each term a separately rounded multiply then add.  The
 * reference accumulates into a zeroed output; this writes every row. */
void orc_aggregate(float* out, const float* x, const int32_t* idx, const int32_t* off,
                   const float* w, int64_t n_out, int64_t f) {
    for (int64_t v = 0; v < n_out; v++) {
        float* o = out + v * f;
        for (int64_t k = 0; k < f; k++) o[k] = 0.0f;
        for (int32_t j = off[v]; j < off[v + 1]; j++) {
            const float* xr = x + (int64_t)idx[j] * f;
            const float wj = w[j];
            for (int64_t k = 0; k < f; k++) {
                float prod = xr[k] * wj;
                o[k] = prod + o[k];
            }
        }
    }
}

/* Per-destination softmax of per-edge scores (ops/cpp/edgesoftmax_op.cc:48-65):
 * max over the segment, then total += expf(x - max) in ascending edge order,
 * then expf(x - max) / total.  The reference handles one scalar per edge; H > 1
 * applies the same recipe to each of the H columns of x[E,H] independently.
 * Empty segments write nothing. */
void orc_edge_softmax(float* out, const float* x, const int32_t* off, int64_t n, int64_t H) {
    for (int64_t v = 0; v < n; v++) {
        int32_t s = off[v], e = off[v + 1];
        if (s >= e) continue;
        for (int64_t h = 0; h < H; h++) {
            float mx = x[(int64_t)s * H + h];
            for (int32_t i = s; i < e; i++)
                if (mx < x[(int64_t)i * H + h]) mx = x[(int64_t)i * H + h];
            float total = 0.0f;
            for (int32_t i = s; i < e; i++) {
                float d = x[(int64_t)i * H + h] - mx;
                out[(int64_t)i * H + h] = d;
                total += expf(d);
            }
            for (int32_t i = s; i < e; i++)
                out[(int64_t)i * H + h] = expf(out[(int64_t)i * H + h]) / total;
        }
    }
}

/* Softmax backward (ops/cpp/edgesoftmaxbackward_op.cc:41-52):
 * dot = sum_seg y*g (ascending), dx = y*g - y*dot.  The reference repeats the
 * same computation deg times (outer loop :44); once gives the same values. */
void orc_edge_softmax_backward(float* out, const float* grad, const float* y, const int32_t* off,
                               int64_t n, int64_t H) {
    for (int64_t v = 0; v < n; v++) {
        int32_t s = off[v], e = off[v + 1];
        for (int64_t h = 0; h < H; h++) {
            float dot = 0.0f;
            for (int32_t i = s; i < e; i++) {
                float p = y[(int64_t)i * H + h] * grad[(int64_t)i * H + h];
                dot += p;
            }
            for (int32_t i = s; i < e; i++) {
                float a = y[(int64_t)i * H + h] * grad[(int64_t)i * H + h];
                float b = y[(int64_t)i * H + h] * dot;
                out[(int64_t)i * H + h] = a - b;
            }
        }
    }
}

/* Node rows copied onto edges in CSC order (ops/cpp/scattertoedge_op.cc:67-87):
 * flag 0 -> row idx[e] (the edge's source), flag 1 -> row v (the segment owner). */
void orc_scatter_to_edge(float* out, const float* x, const int32_t* idx, const int32_t* off,
                         int64_t n, int64_t f, int flag) {
    for (int64_t v = 0; v < n; v++)
        for (int32_t e = off[v]; e < off[v + 1]; e++) {
            const float* xr = x + (flag == 0 ? (int64_t)idx[e] : v) * f;
            for (int64_t k = 0; k < f; k++) out[(int64_t)e * f + k] = xr[k];
        }
}

/* Edge messages summed onto nodes (ops/cpp/edgetovertex_op.cc:35-55): flag 1 adds
 * edge e of segment v to row v, flag 0 adds it to row idx[e]; edges visited in
 * ascending order.  Writes every output row (zero for rows nothing reaches). */
void orc_edge_to_vertex(float* out, const float* msg, const int32_t* idx, const int32_t* off,
                        int64_t n, int64_t f, int flag) {
    memset(out, 0, sizeof(float) * (size_t)(n * f));
    for (int64_t v = 0; v < n; v++)
        for (int32_t e = off[v]; e < off[v + 1]; e++) {
            float* o = out + (flag == 0 ? (int64_t)idx[e] : v) * f;
            for (int64_t k = 0; k < f; k++) o[k] = o[k] + msg[(int64_t)e * f + k];
        }
}

/* Multi-head attention layer over CSC in-edges, following the composition of
 * nn/conv/gat_conv.py:67-83 (scatter src/dst rows to edges, logits through
 * leaky_relu(.,0.2), per-destination softmax, weight the source rows, sum per
 * destination) without materialising the per-edge tensors.  h is [n, H*D];
 * a_src/a_dst are [H, D].  With H = 1 this is exactly the reference layer after
 * its dense transform.  Logit for edge e: sum over the concatenated
 * [h_src, h_dst] . [a_src, a_dst] accumulated left to right as a matmul row. */
void orc_gat_aggregate(float* out, const float* h, const float* a_src, const float* a_dst,
                       const int32_t* idx, const int32_t* off, int64_t n, int64_t H, int64_t D,
                       float slope) {
    const int64_t C = H * D;
    int32_t maxdeg = 0;
    for (int64_t v = 0; v < n; v++)
        if (off[v + 1] - off[v] > maxdeg) maxdeg = off[v + 1] - off[v];
    float* logit = (float*)malloc(sizeof(float) * (size_t)(maxdeg > 0 ? maxdeg : 1));
    for (int64_t v = 0; v < n; v++) {
        int32_t s = off[v], e = off[v + 1];
        float* o = out + v * C;
        for (int64_t k = 0; k < C; k++) o[k] = 0.0f;
        if (s >= e) continue;
        for (int64_t hd = 0; hd < H; hd++) {
            for (int32_t i = s; i < e; i++) {
                const float* hs = h + (int64_t)idx[i] * C + hd * D;
                const float* ht = h + v * C + hd * D;
                float acc = 0.0f;
                for (int64_t d = 0; d < D; d++) acc += hs[d] * a_src[hd * D + d];
                for (int64_t d = 0; d < D; d++) acc += ht[d] * a_dst[hd * D + d];
                logit[i - s] = acc > 0.0f ? acc : acc * slope;
            }
            float mx = logit[0];
            for (int32_t i = 1; i < e - s; i++)
                if (mx < logit[i]) mx = logit[i];
            float total = 0.0f;
            for (int32_t i = 0; i < e - s; i++) {
                logit[i] -= mx;
                total += expf(logit[i]);
            }
            for (int32_t i = s; i < e; i++) {
                float alpha = expf(logit[i - s]) / total;
                const float* hs = h + (int64_t)idx[i] * C + hd * D;
                for (int64_t d = 0; d < D; d++) o[hd * D + d] = o[hd * D + d] + hs[d] * alpha;
            }
        }
    }
    free(logit);
}

/* Symmetric normalisation with self-loops (nn/conv/gcn_conv.py:18-37 and
 * utils/loop.py:120-134).  Input COO (src,dst,w) of E0 edges; w == NULL means
 * unit weights.  Existing (i,i) edges are dropped and their weight moved onto the
 * appended loop (last one wins, as an indexed assignment does); loops for nodes
 * 0..n-1 are appended in node order.  Outputs hold E = E0 - #loops + n entries
 * (capacity E0 + n).  deg[dst] accumulates in list order; weights are
 * (dis[src] * w) * dis[dst] with dis = deg^-1/2 in fp32.  Returns E. */
int64_t orc_gcn_norm(const int32_t* src, const int32_t* dst, const float* w, int64_t E0, int32_t n,
                     int32_t* out_src, int32_t* out_dst, float* out_w, int add_self_loops) {
    int64_t m = 0;
    int64_t E;
    if (add_self_loops) {
        for (int64_t i = 0; i < E0; i++)
            if (src[i] != dst[i]) {
                out_src[m] = src[i];
                out_dst[m] = dst[i];
                out_w[m] = w ? w[i] : 1.0f;
                m++;
            }
        for (int32_t v = 0; v < n; v++) {
            out_src[m + v] = v;
            out_dst[m + v] = v;
            out_w[m + v] = 1.0f;
        }
        for (int64_t i = 0; i < E0; i++)
            if (src[i] == dst[i]) out_w[m + src[i]] = w ? w[i] : 1.0f;
        E = m + n;
    } else {
        /* add_self_loops=False (nn/conv/gcn_conv.py:25): the list is normalised as given */
        for (int64_t i = 0; i < E0; i++) {
            out_src[i] = src[i];
            out_dst[i] = dst[i];
            out_w[i] = w ? w[i] : 1.0f;
        }
        E = E0;
    }
    float* deg = (float*)calloc((size_t)(n > 0 ? n : 1), sizeof(float));
    for (int64_t i = 0; i < E; i++) deg[out_dst[i]] += out_w[i];
    for (int32_t v = 0; v < n; v++) deg[v] = powf(deg[v], -0.5f);
    for (int64_t i = 0; i < E; i++) {
        float t = deg[out_src[i]] * out_w[i];
        out_w[i] = t * deg[out_dst[i]];
    }
    free(deg);
    return E;
}

/* Mirror + sort by (row, col) + drop duplicate pairs (ops/cpp/toundirected_op.cc:33-63).
 * The reference sorts with std::sort (not stable), so WHICH duplicate's attribute
 * survives is unspecified there; here the first in mirrored-list order survives.
 * Outputs need room for 2*E entries; returns the new edge count. */
typedef struct { int32_t r, c; float a; int64_t pos; } orc_edge_t;
static int orc_edge_cmp(const void* pa, const void* pb) {
    const orc_edge_t* a = (const orc_edge_t*)pa;
    const orc_edge_t* b = (const orc_edge_t*)pb;
    if (a->r != b->r) return a->r < b->r ? -1 : 1;
    if (a->c != b->c) return a->c < b->c ? -1 : 1;
    return a->pos < b->pos ? -1 : (a->pos > b->pos ? 1 : 0);
}
int64_t orc_to_undirected(const int32_t* src, const int32_t* dst, const float* attr, int64_t E,
                          int32_t* out_src, int32_t* out_dst, float* out_attr) {
    orc_edge_t* ed = (orc_edge_t*)malloc(sizeof(orc_edge_t) * (size_t)(2 * E > 0 ? 2 * E : 1));
    for (int64_t i = 0; i < E; i++) {
        ed[2 * i] = (orc_edge_t){src[i], dst[i], attr[i], 2 * i};
        ed[2 * i + 1] = (orc_edge_t){dst[i], src[i], attr[i], 2 * i + 1};
    }
    qsort(ed, (size_t)(2 * E), sizeof(orc_edge_t), orc_edge_cmp);
    int64_t m = 0;
    for (int64_t i = 0; i < 2 * E; i++) {
        if (m > 0 && out_src[m - 1] == ed[i].r && out_dst[m - 1] == ed[i].c) continue;
        out_src[m] = ed[i].r;
        out_dst[m] = ed[i].c;
        out_attr[m] = ed[i].a;
        m++;
    }
    free(ed);
    return m;
}

/* ---- neighbour-sampling operators ------------------------------------------------------------
 * layer column counts (ops/cpp/gpuinitco_op.cc:37-52, the CUDA kernel; the CPU body is empty):
 * out[i+1] = min(in-degree of dst[i], fanout); out[0] is left as the caller set it. */
void orc_sample_counts(const int32_t* dst, int64_t n_dst, const int32_t* g_off, int32_t fanout, int32_t* out) {
    for (int64_t i = 0; i < n_dst; i++) {
        const int32_t deg = g_off[dst[i] + 1] - g_off[dst[i]];
        out[i + 1] = deg < fanout ? deg : fanout;
    }
}

/* CSC -> CSR over explicit id lists (ops/cpp/csctocsr_op.cc:26-80): row r of the result belongs to
 * src_ids[r]; column values are dst_ids[column]; entries whose source id is not listed are dropped;
 * inside a row the entries keep the CSC traversal order.  row_off must be zero-filled.  Returns the
 * number of entries written. */
int64_t orc_csc_to_csr(const int32_t* col_off, const int32_t* row_idx, int64_t n_dst, const int32_t* dst_ids,
                       const int32_t* src_ids, int64_t n_src, int32_t max_id, int32_t* row_off, int32_t* col_idx) {
    int32_t* where = (int32_t*)malloc(sizeof(int32_t) * (size_t)(max_id + 1));
    for (int32_t i = 0; i <= max_id; i++) where[i] = -1;
    for (int64_t i = 0; i < n_src; i++) where[src_ids[i]] = (int32_t)i;
    for (int64_t i = 0; i < n_dst; i++)
        for (int32_t j = col_off[i]; j < col_off[i + 1]; j++) {
            const int32_t r = row_idx[j] <= max_id ? where[row_idx[j]] : -1;
            if (r >= 0) row_off[r + 1]++;
        }
    for (int64_t i = 1; i <= n_src; i++) row_off[i] += row_off[i - 1];
    int32_t* cur = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n_src > 0 ? n_src : 1));
    for (int64_t i = 0; i < n_src; i++) cur[i] = row_off[i];
    for (int64_t i = 0; i < n_dst; i++)
        for (int32_t j = col_off[i]; j < col_off[i + 1]; j++) {
            const int32_t r = row_idx[j] <= max_id ? where[row_idx[j]] : -1;
            if (r >= 0) col_idx[cur[r]++] = dst_ids[i];
        }
    const int64_t kept = row_off[n_src];
    free(cur);
    free(where);
    return kept;
}

/* symmetric degree weights of a sampled layer (ops/cpp/getweight_op.cc:37-84): in-degree of
 * dst_ids[i] += length of column i, out-degree of every listed source += 1 per entry,
 * w = 1 / (sqrtf(out[src]) * sqrtf(in[dst])). */
void orc_get_weight(int32_t vtx_size, const int32_t* dst_ids, int64_t n_dst, const int32_t* col_off, const int32_t* row_idx,
                    float* out_w) {
    int32_t* ins = (int32_t*)calloc((size_t)(vtx_size > 0 ? vtx_size : 1), sizeof(int32_t));
    int32_t* outs = (int32_t*)calloc((size_t)(vtx_size > 0 ? vtx_size : 1), sizeof(int32_t));
    for (int64_t i = 0; i < n_dst; i++) {
        ins[dst_ids[i]] += col_off[i + 1] - col_off[i];
        for (int32_t j = col_off[i]; j < col_off[i + 1]; j++) outs[row_idx[j]] += 1;
    }
    for (int64_t i = 0; i < n_dst; i++)
        for (int32_t j = col_off[i]; j < col_off[i + 1]; j++)
            out_w[j] = 1 / (sqrtf((float)outs[row_idx[j]]) * sqrtf((float)ins[dst_ids[i]]));
    free(ins);
    free(outs);
}
