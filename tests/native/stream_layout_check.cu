// CPU check of the single-session decode kernel's layout arithmetic (csrc/decode_stream_layout.hpp): built with nvcc, run on the
// host only - no CUDA call is made.  Prints one line per case and exits non-zero on the first violated property.
#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "decode_stream_layout.hpp"

using namespace rsv;

static int failures = 0;
#define CHECK(cond, ...)                     \
    do {                                     \
        if (!(cond)) {                       \
            std::printf("FAIL: " __VA_ARGS__); \
            std::printf("\n");               \
            ++failures;                      \
        }                                    \
    } while (0)

static void check_shape(const char* name, DsShape s, int G) {
    DsLayout lay;
    std::string why;
    const bool ok = ds_layout(s, G, lay, why);
    CHECK(ok, "%s on %d SMs: refused: %s", name, G, why.c_str());
    if (!ok) return;
    CHECK(lay.smem <= 227u * 1024u && lay.ring_bytes % 128 == 0 && lay.ring_bytes >= 64 * 1024, "%s: shared memory %zu, ring %d", name, lay.smem, lay.ring_bytes);
    for (int layer0 = 0; layer0 < 2; ++layer0) {
        DsEntry ents[DSE_COUNT];
        ds_layer_entries(s, G, true, ents);  // the plan is always built from a layer with a v gate; layer 0 skips those chunks
        const DsEntry head_e = ds_head_entry(s, G);
        std::vector<std::vector<char>> seen(DSE_COUNT + 1);
        for (int e = 0; e <= DSE_COUNT; ++e) seen[e].assign((size_t)(e == DSE_COUNT ? head_e.M : ents[e].M), 0);
        auto plan = std::make_unique<DsPlan>();
        for (int c = 0; c < G; ++c) {
            CHECK(ds_build_plan(*plan, ents, head_e, c, G, 0u), "%s: CTA %d: chunk table overflow", name, c);
            for (int e = 0; e <= DSE_COUNT; ++e)
                for (int r = plan->er0[e]; r < plan->er0[e] + plan->en[e]; ++r) {
                    CHECK(r >= 0 && r < (int)seen[e].size() && !seen[e][r], "%s: CTA %d: row %d of matrix %d handed out twice or outside", name, c, r, e);
                    if (r >= 0 && r < (int)seen[e].size()) seen[e][r] = 1;
                }
            // the chunks of the v-gate projection, skipped in layer 0, are the first of the CTA's phase-1 list
            const int nv1 = plan->phn[DSP_P1] - plan->phn_l0;
            for (int k = 0; k < plan->phn[DSP_P1]; ++k) {
                const bool is_v1 = (plan->ctab[plan->ph0[DSP_P1] + k].e_flags_row0 & 0xFF) == DSE_V1;
                CHECK(is_v1 == (k < nv1), "%s: CTA %d: v-gate chunks are not the first %d of phase 1", name, c, nv1);
            }
            long long bytes = 0;
            for (int ph = DSP_P1; ph <= DSP_P5; ++ph)
                for (int k = plan->ph0[ph]; k < plan->ph0[ph] + plan->phn[ph]; ++k) {
                    const DsChunk& ch = plan->ctab[k];
                    const int nr = ch.nr_steps & 0xFFFF, steps = ch.nr_steps >> 16, e = ch.e_flags_row0 & 0xFF;
                    CHECK(nr >= 1 && nr <= kDsTileRows && steps >= 2 && steps % 2 == 0, "%s: CTA %d: chunk %d: %d rows, %d steps", name, c, k, nr, steps);
                    CHECK(ch.stride == ents[e].piece_bytes + kDsPad && ch.cb >= nr * ch.stride && ch.cb % 16 == 0, "%s: CTA %d: chunk %d: bytes", name, c, k);
                    bytes += ch.cb;
                }
            CHECK(bytes + 128LL * s.mids() <= lay.wslot, "%s: CTA %d: %lld bytes of rows do not fit the %lld-byte region", name, c, bytes, lay.wslot);
            // a head's three chunks: resident together, or the first alone and then the other two, plus one wrap's waste
            const int a = 64 * (s.wm + s.am) * 2, b = 64 * s.vm * 2 + 32 * s.gm * 2, cc = 32 * s.gm * 2;
            if (lay.head_early)
                CHECK(2 * a <= lay.ring_bytes && b + cc + std::max(b, cc) <= lay.ring_bytes, "%s: head chunks (%d, %d, %d) against a ring of %d", name, a, b, cc, lay.ring_bytes);
            else
                CHECK(a + b + cc + std::max(a, std::max(b, cc)) <= lay.ring_bytes, "%s: head chunks (%d, %d, %d) against a ring of %d", name, a, b, cc, lay.ring_bytes);
        }
        for (int e = 0; e <= DSE_COUNT; ++e)
            for (size_t r = 0; r < seen[e].size(); ++r) CHECK(seen[e][r], "%s: row %zu of matrix %d belongs to no CTA", name, r, e);
        // every head has a CTA of its own in every layer
        for (int l = 0; l < 3; ++l) {
            std::vector<int> owner((size_t)s.H, -1);
            for (int c = 0; c < G; ++c) {
                const int h = ds_head_of_cta(c, l, s.H, G);
                if (h >= 0) {
                    CHECK(h < s.H && owner[h] < 0, "%s: layer %d: head %d on two CTAs", name, l, h);
                    if (h < s.H) owner[h] = c;
                }
            }
            for (int h = 0; h < s.H; ++h) CHECK(owner[h] >= 0, "%s: layer %d: head %d has no CTA", name, l, h);
        }
    }
    std::printf("ok %-28s SMs %3d  kernel<%d>  ring %6d B  region %8lld B%s\n", name, G, lay.cmax, lay.ring_bytes, lay.wslot, lay.head_early ? "  (first head chunk released early)" : "");
}

static void check_refused(const char* name, DsShape s, int G, const char* expect) {
    DsLayout lay;
    std::string why;
    const bool ok = ds_layout(s, G, lay, why);
    CHECK(!ok && why.find(expect) != std::string::npos, "%s: expected a refusal mentioning '%s', got %s '%s'", name, expect, ok ? "acceptance" : "refusal", why.c_str());
    if (!ok) std::printf("ok %-28s refused: %s\n", name, why.c_str());
}

int main() {
    const DsShape tiny{4, 512, 2048, 4096, 8, 32, 32, 16, 64, 0, 0};
    const DsShape b3{32, 2560, 10240, 65536, 40, 96, 96, 64, 320, 1, 0};
    const DsShape b7{32, 4096, 16384, 65536, 64, 128, 128, 96, 480, 1, 0};
    for (int fmt = 0; fmt < 3; ++fmt)
        for (int hf = 0; hf < 3; hf += 2) {
            DsShape t = tiny, m = b3, l = b7;
            t.fmt = m.fmt = l.fmt = fmt;
            t.head_fmt = m.head_fmt = l.head_fmt = hf;
            const std::string tag = " fmt " + std::to_string(fmt) + " head " + std::to_string(hf);
            check_shape(("tiny" + tag).c_str(), t, 148);
            check_shape(("3b" + tag).c_str(), m, 148);
            if (fmt == 0 && hf == 0)  // 8192-byte rows everywhere: more chunks per SM than the table holds - the engine takes the multi-kernel path
                check_refused(("7b" + tag).c_str(), l, 148, "too many chunks");
            else
                check_shape(("7b" + tag).c_str(), l, 148);
        }
    check_shape("3b on 132 SMs", b3, 132);
    check_refused("3b on 64 SMs", b3, 64, "too many channels per SM");
    check_shape("1.5b-like", DsShape{24, 2048, 8192, 65536, 32, 96, 96, 64, 256, 2, 2}, 148);
    check_shape("0.1b-like", DsShape{12, 768, 3072, 65536, 12, 64, 64, 32, 128, 0, 0}, 148);
    check_refused("more heads than SMs", b7, 48, "more heads than SMs");
    check_refused("n_embd 2600", DsShape{2, 2600, 10400, 4096, 40, 96, 96, 64, 320, 0, 0}, 148, "multiple of 128");
    check_refused("ffn 3 n_embd", DsShape{2, 2560, 7680, 4096, 40, 96, 96, 64, 320, 0, 0}, 148, "ffn_hidden");
    check_refused("rank 100", DsShape{2, 2560, 10240, 4096, 40, 100, 96, 64, 320, 0, 0}, 148, "multiples of 8");
    check_refused("huge gate rank", DsShape{2, 4096, 16384, 4096, 64, 128, 128, 96, 2048, 0, 0}, 148, "back-projection rows do not fit");
    check_refused("13b-like", DsShape{40, 5120, 20480, 65536, 80, 128, 128, 96, 480, 1, 0}, 148, "at most 4096");
    if (failures) {
        std::printf("%d failures\n", failures);
        return 1;
    }
    std::printf("all layout checks passed\n");
    return 0;
}
