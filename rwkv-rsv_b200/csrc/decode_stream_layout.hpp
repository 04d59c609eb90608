// Host-side layout of the single-session weight-streaming decode kernel (decode_stream.cuh): which CTA owns which rows of
// which matrix, how rows are cut into chunks, how much shared memory the ring gets, and every capacity the kernel's fixed-size
// tables assume.  Pure arithmetic on the model's shape - no CUDA call, no device memory - so that it can be checked on a machine
// without a GPU; the engine fills in the pointers afterwards.
#pragma once
#include <algorithm>
#include <memory>
#include <string>
#include <vector>

#include "decode_stream.cuh"

namespace rsv {

// Weight formats: 0 fp16, 1 int8 with one (scale, zero) per output row, 2 int8 with one per row and group of 128 weights.
struct DsShape {
    int L, C, F, V, H;
    int wm, am, vm, gm;  // rank dimensions of the decay, a, v-gate and output-gate projections
    int fmt, head_fmt;   // format of the six big matrices of a layer, and of the vocabulary head
    int mids() const { return wm + am + vm + gm; }
};

struct DsLayout {
    int cmax = 0;        // template instance of the kernel
    int vec_floats = 0;  // operand area
    int ring_bytes = 0;
    size_t smem = 0;
    bool head_early = false;
    long long wslot = 0, hslot = 0;  // bytes of the consumption-order weight copy per (layer, CTA) and of the head's per CTA
};

// Sizes of one matrix [M, K]: pieces of at most max_piece bytes, each a multiple of 128 bytes; all CTAs, no pointers.
inline DsEntry ds_size_entry(int M, int K, int fmt, int G, int xvec, int out, int out_off, int max_piece = kDsMaxPiece) {
    DsEntry e{};
    const int row_bytes = fmt ? K : 2 * K;
    int np = (row_bytes + max_piece - 1) / max_piece;
    while (np <= row_bytes / 128 && row_bytes % (np * 128)) ++np;
    e.M = M;
    e.row_stride = row_bytes;
    e.piece_bytes = row_bytes / std::max(np, 1);
    e.npieces = np;
    e.is_i8 = fmt;
    e.xvec = xvec;
    e.out = out;
    e.out_off = out_off;
    e.cta0 = 0;
    e.ncta = G;
    return e;
}

// The ten matrices of a layer with their CTA groups (layer 0 has no v-gate projection).
inline void ds_layer_entries(const DsShape& s, int G, bool has_vgate, DsEntry (&e)[DSE_COUNT]) {
    const int C = s.C, F = s.F;
    // operand vectors of phase 1: 0 = the shifted input of the CTA's big matrix (receptance, key or value), 1 = that of its rank
    // projection
    e[DSE_W1] = ds_size_entry(s.wm, C, 0, G, 1, DSO_MID_TANH, 0);
    e[DSE_A1] = ds_size_entry(s.am, C, 0, G, 1, DSO_MID, s.wm);
    e[DSE_G1] = ds_size_entry(s.gm, C, 0, G, 1, DSO_MID_SIG, s.wm + s.am + s.vm);
    e[DSE_V1] = ds_size_entry(s.vm, C, 0, G, 1, DSO_MID, s.wm + s.am);
    // The rows of the four rank projections go to disjoint groups of CTAs, sized by their row counts, so that a CTA builds the
    // shifted input of one of them only.
    {
        const int order[4] = {DSE_W1, DSE_A1, DSE_V1, DSE_G1};
        const int rows_of_e[4] = {s.wm, s.am, s.vm, s.gm};
        int c0 = 0, rows_left = s.mids(), ctas_left = G;
        for (int i = 0; i < 4; ++i) {
            DsEntry& x = e[order[i]];
            int nc = i == 3 ? ctas_left : std::max(1, (int)((long long)ctas_left * rows_of_e[i] / std::max(rows_left, 1)));
            nc = std::max(1, std::min(nc, ctas_left - (3 - i)));
            x.cta0 = c0;
            x.ncta = nc;
            c0 += nc;
            ctas_left -= nc;
            rows_left -= rows_of_e[i];
        }
    }
    if (!has_vgate) e[DSE_V1].M = 0;
    e[DSE_WR] = ds_size_entry(C, C, s.fmt, G, 0, DSO_R, 0, kDsLayerPiece);
    e[DSE_WK] = ds_size_entry(C, C, s.fmt, G, 0, DSO_K, 0, kDsLayerPiece);
    e[DSE_WV] = ds_size_entry(C, C, s.fmt, G, 0, DSO_V, 0, kDsLayerPiece);
    e[DSE_WO] = ds_size_entry(C, C, s.fmt, G, 0, DSO_XADD, 0, kDsLayerPiece);
    e[DSE_WFK] = ds_size_entry(F, C, s.fmt, G, 0, DSO_H, 0, kDsLayerPiece);
    e[DSE_WFV] = ds_size_entry(C, F, s.fmt, G, 0, DSO_XADD, 0, kDsLayerPiece);
    // receptance, key and value go to three disjoint thirds of the CTAs (all rows of one matrix over a third), so that a CTA
    // builds the shifted input and the fixed-point digits of one of them instead of all three, and its rows make full tiles
    const int third = G / 3;
    e[DSE_WR].cta0 = 0;
    e[DSE_WR].ncta = third;
    e[DSE_WK].cta0 = third;
    e[DSE_WK].ncta = third;
    e[DSE_WV].cta0 = 2 * third;
    e[DSE_WV].ncta = G - 2 * third;
}

inline DsEntry ds_head_entry(const DsShape& s, int G) { return ds_size_entry(s.V, s.C, s.head_fmt, G, 0, DSO_LOGITS, 0); }

// Everything the kernel assumes about a shape on a GPU of G SMs, checked exactly (every CTA's plan is built).  Returns false and
// says why when the kernel cannot run the shape; the caller then takes another path.
inline bool ds_layout(const DsShape& s, int G, DsLayout& out, std::string& why) {
    auto fail = [&](const std::string& w) {
        why = w;
        return false;
    };
    const int C = s.C, F = s.F, H = s.H;
    out = DsLayout{};
    for (int c : {512, 1024, 2048, 2560, 4096})
        if (!out.cmax && C <= c) out.cmax = c;
    if (C <= 0 || C % 128 || !out.cmax) return fail("n_embd must be a multiple of 128 and at most 4096");
    if (C != H * 64) return fail("n_embd is not 64 x heads");
    if (F != 4 * C) return fail("ffn_hidden is not 4 n_embd");
    if (G < 3) return fail("fewer than three SMs");
    if (H > G) return fail("more heads than SMs");
    if (s.wm <= 0 || s.am <= 0 || s.vm <= 0 || s.gm <= 0 || s.wm % 8 || s.am % 8 || s.vm % 8 || s.gm % 8) return fail("rank dimensions must be positive multiples of 8");
    if (s.fmt < 0 || s.fmt > 2 || s.head_fmt < 0 || s.head_fmt > 2) return fail("unknown weight format");
    if (F / 128 > kDsMaxGroups) return fail("reduction longer than 16384");
    // shared memory: ring + operand area + fixed part + rank-space vector
    const size_t budget = 227 * 1024;
    out.vec_floats = std::max(4 * C, F);
    const size_t fixed = (size_t)out.vec_floats * 4 + sizeof(DsShared) + (size_t)s.mids() * 4 + 256;
    if (fixed + 64 * 1024 > budget) return fail("operand area does not fit in shared memory");
    out.ring_bytes = (int)((budget - fixed) / 128 * 128);
    out.smem = (size_t)out.ring_bytes + fixed;
    const int R = out.ring_bytes;
    // A head's back-projection rows come as three chunks (w2 + a2; v2 + half of g2; the other half of g2).  The ring hands out
    // contiguous space in order, so what must be resident together needs its bytes plus one wrap's waste (< the largest chunk):
    // all three when the head phase returns them together, else the first alone and then the other two.
    const int hb_a = 64 * (s.wm + s.am) * 2, hb_b = 64 * s.vm * 2 + 32 * s.gm * 2, hb_c = 32 * s.gm * 2;
    out.head_early = hb_a + hb_b + hb_c + std::max({hb_a, hb_b, hb_c}) > R;
    if (out.head_early && std::max(2 * hb_a, hb_b + hb_c + std::max(hb_b, hb_c)) > R) return fail("a head's back-projection rows do not fit in the shared-memory ring");
    // every CTA's plan, layer with a v gate (the larger one)
    DsEntry ents[DSE_COUNT];
    ds_layer_entries(s, G, true, ents);
    const DsEntry head_e = ds_head_entry(s, G);
    for (int i = 0; i < DSE_COUNT; ++i)
        if (ents[i].piece_bytes % 128 || ents[i].piece_bytes > kDsMaxPiece || ents[i].npieces < 1) return fail("a weight row does not split into pieces of a multiple of 128 bytes");
    if (head_e.piece_bytes % 128 || head_e.piece_bytes > kDsMaxPiece) return fail("a head row does not split into pieces of a multiple of 128 bytes");
    for (int e : {DSE_W1, DSE_A1, DSE_G1, DSE_V1})
        if (ents[e].npieces * ents[e].piece_bytes != 2 * C) return fail("rank projections must be fp16 [mid, n_embd]");
    auto plan = std::make_unique<DsPlan>();
    std::vector<int> next_row(DSE_COUNT + 1, 0);  // rows must be handed out in order, without gaps, once
    const int first[DSP_COUNT] = {DSE_W1, DSE_WO, DSE_WFK, DSE_WFV, DSE_COUNT}, last[DSP_COUNT] = {DSE_WV, DSE_WO, DSE_WFK, DSE_WFV, DSE_COUNT};
    for (int c = 0; c < G; ++c) {
        if (!ds_build_plan(*plan, ents, head_e, c, G, 0u)) return fail("too many chunks per SM for the chunk table");
        int rank_entries = 0, big_entries = 0;
        for (int e = DSE_W1; e <= DSE_V1; ++e) rank_entries += plan->en[e] > 0;
        for (int e = DSE_WR; e <= DSE_WV; ++e) big_entries += plan->en[e] > 0;
        if (rank_entries > 1 || big_entries != 1) return fail("a CTA must own rows of one rank projection at most and of exactly one of receptance, key, value");
        if (plan->en[DSE_WO] != plan->en[DSE_WFV] || plan->er0[DSE_WO] != plan->er0[DSE_WFV]) return fail("att.output and ffn.value rows of a CTA differ (they are its slice of x)");
        if (plan->en[DSE_WO] > kDsMaxSlice) return fail("too many channels per SM");
        long long rows = 0, hd = 0;
        for (int ph = 0; ph < DSP_COUNT; ++ph) {
            int tiles = 0, part = 0, staged = 0;
            for (int e = first[ph]; e <= last[ph]; ++e) {
                const DsEntry& E = e == DSE_COUNT ? head_e : ents[e];
                const int n = plan->en[e];
                if (n <= 0) continue;
                const int t = (n + kDsTileRows - 1) / kDsTileRows;
                tiles += t;
                part += t * E.npieces * kDsTileRows * (E.is_i8 == 1 ? 8 : 4);
                if (E.is_i8 == 1) staged += n;
            }
            if (tiles > kDsMaxTiles) return fail("too many tiles per SM");
            if (part > kDsPartBytes) return fail("partial sums of a phase do not fit in shared memory");
            if (staged > kDsMaxRows) return fail("too many rows per SM");
            for (int k = plan->ph0[ph]; k < plan->ph0[ph] + plan->phn[ph]; ++k) {
                const DsChunk& ch = plan->ctab[k];
                if (ch.cb % 16 || 2 * ch.cb > R) return fail("a chunk of rows does not fit twice in the shared-memory ring");
                (ph == DSP_HEAD ? hd : rows) += ch.cb;
            }
        }
        for (int e = 0; e <= DSE_COUNT; ++e) {
            const DsEntry& E = e == DSE_COUNT ? head_e : ents[e];
            if (plan->en[e] <= 0) continue;
            // CTAs are visited in index order; an entry's virtual order starts at cta0, so its rows need not come in CTA order:
            // only check that ranges are inside the matrix (coverage is summed below)
            if (plan->er0[e] < 0 || plan->er0[e] + plan->en[e] > E.M) return fail("a CTA's rows lie outside the matrix");
            next_row[e] += plan->en[e];
        }
        out.wslot = std::max(out.wslot, rows);
        out.hslot = std::max(out.hslot, hd);
    }
    for (int e = 0; e <= DSE_COUNT; ++e)
        if (next_row[e] != (e == DSE_COUNT ? head_e.M : ents[e].M)) return fail("the CTAs' rows do not add up to the matrix");
    out.wslot += 128LL * s.mids();  // a head's back-projection rows
    out.wslot = (out.wslot + 255) / 256 * 256;
    out.hslot = (out.hslot + 255) / 256 * 256;
    return true;
}

}  // namespace rsv
