// Self-test of the cache-management kernel bodies (csrc/cache_ops_body.h) under AddressSanitizer:
// randomized and adversarial cases on heap buffers of exactly the stated sizes, every (CTA, thread) of
// the grid emulated in turn, results compared with plain loops.  An out-of-bounds read or write of a
// kernel body aborts here, on the CPU.  Build: g++ -fsanitize=address,undefined (build.py).
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include "../../ascend-transformer-boost_b200/csrc/cache_ops_body.h"

using namespace atb_b200;

namespace {

uint64_t g_state = 0x9e3779b97f4a7c15ull;
uint32_t rnd()
{
    g_state ^= g_state << 13;
    g_state ^= g_state >> 7;
    g_state ^= g_state << 17;
    return (uint32_t)(g_state >> 32);
}
int rnd_in(int lo, int hi) { return lo + (int)(rnd() % (uint32_t)(hi - lo + 1)); }

// 16-byte aligned heap buffer of exactly n bytes (ASan guards both ends)
struct Buf {
    uint8_t *p = nullptr;
    size_t n = 0;
    explicit Buf(size_t bytes, bool align16 = true) : n(bytes)
    {
        if (align16) {
            if (posix_memalign(reinterpret_cast<void **>(&p), 16, bytes ? bytes : 16) != 0) {
                std::abort();
            }
        } else {
            raw = static_cast<uint8_t *>(std::malloc(bytes + 1));
            p = raw + 1; // deliberately odd
        }
        for (size_t i = 0; i < bytes; ++i) {
            p[i] = (uint8_t)rnd();
        }
    }
    ~Buf() { std::free(raw ? raw : p); }
    uint8_t *raw = nullptr;
};

int failures = 0;
void expect(bool ok, const char *what, int case_id)
{
    if (!ok) {
        std::fprintf(stderr, "FAIL %s (case %d)\n", what, case_id);
        ++failures;
    }
}

void test_block_copy(int case_id)
{
    const int blocks = rnd_in(2, 40);
    const bool odd = rnd() % 4 == 0;                       // byte path: sizes / pointers not multiples of 16
    const int64_t kb = odd ? rnd_in(1, 200) : 16 * rnd_in(1, 40);
    const int64_t vb = odd ? rnd_in(1, 200) : 16 * rnd_in(1, 40);
    const bool has_v = rnd() % 5 != 0;
    const int n_src = rnd_in(1, blocks / 2 > 0 ? blocks / 2 : 1);
    const int n_dst = rnd_in(n_src, blocks);
    Buf k((size_t)blocks * kb, !odd), v((size_t)blocks * vb, !odd);
    std::vector<int32_t> src(n_src), dst(n_dst), cum(n_src);
    // destinations: distinct blocks that are not sources (as the operation requires), plus some invalid ids
    std::vector<int> is_src(blocks, 0);
    for (int i = 0; i < n_src; ++i) {
        src[i] = rnd_in(0, blocks - 1);
        is_src[src[i]] = 1;
    }
    std::vector<int> free_blocks;
    for (int b = 0; b < blocks; ++b) {
        if (!is_src[b]) {
            free_blocks.push_back(b);
        }
    }
    for (int j = 0; j < n_dst; ++j) {
        if (!free_blocks.empty() && rnd() % 8 != 0) {
            const int pick = rnd_in(0, (int)free_blocks.size() - 1);
            dst[j] = free_blocks[pick];
            free_blocks.erase(free_blocks.begin() + pick);
        } else {
            dst[j] = (rnd() % 2) ? -1 - (int)(rnd() % 5) : blocks + (int)(rnd() % 5); // must be skipped
        }
    }
    if (rnd() % 6 == 0) {
        src[rnd_in(0, n_src - 1)] = blocks + 3; // an invalid source: its destinations stay untouched
    }
    int acc = 0;
    for (int i = 0; i < n_src; ++i) {
        acc += rnd_in(0, 2 * n_dst / n_src + 1);
        cum[i] = acc;
    }
    if (rnd() % 2) {
        cum[n_src - 1] = n_dst;
    }
    // reference
    std::vector<uint8_t> kref(k.p, k.p + k.n), vref(v.p, v.p + v.n);
    {
        const std::vector<uint8_t> k0 = kref, v0 = vref;
        int start = 0;
        for (int i = 0; i < n_src; ++i) {
            const int end = cum[i] < n_dst ? cum[i] : n_dst;
            for (int j = start > 0 ? start : 0; j < end; ++j) {
                const int64_t s = src[i], d = dst[j];
                if (s < 0 || s >= blocks || d < 0 || d >= blocks || s == d) {
                    continue;
                }
                std::memcpy(&kref[d * kb], &k0[s * kb], kb);
                if (has_v) {
                    std::memcpy(&vref[d * vb], &v0[s * vb], vb);
                }
            }
            start = cum[i] > start ? cum[i] : start;
        }
    }
    BlockCopyArgs a{};
    a.k_cache = k.p;
    a.v_cache = has_v ? v.p : nullptr;
    a.src = src.data();
    a.dst = dst.data();
    a.cum = cum.data();
    a.n_src = n_src;
    a.n_dst = n_dst;
    a.k_block_bytes = kb;
    a.v_block_bytes = has_v ? vb : 0;
    a.num_blocks = blocks;
    a.chunks = rnd_in(1, 5);
    a.vec16 = !odd && kb % 16 == 0 && a.v_block_bytes % 16 == 0;
    const int threads = rnd_in(1, 7);
    for (int64_t cta = 0; cta < (int64_t)n_dst * a.chunks; ++cta) {
        for (int tid = 0; tid < threads; ++tid) {
            block_copy_body(a, cta, tid, threads);
        }
    }
    expect(std::memcmp(k.p, kref.data(), k.n) == 0, "block_copy key cache", case_id);
    expect(std::memcmp(v.p, vref.data(), v.n) == 0, "block_copy value cache", case_id);
}

void test_paged_cache_load(int case_id)
{
    const int blocks = rnd_in(1, 20), bs = 1 << rnd_in(0, 5), batch = rnd_in(1, 8), cols = rnd_in(1, 9);
    const bool odd = rnd() % 4 == 0;
    const int64_t krow = odd ? rnd_in(1, 70) : 16 * rnd_in(1, 12), vrow = odd ? rnd_in(1, 70) : 16 * rnd_in(1, 12);
    const bool has_v = rnd() % 5 != 0, has_starts = rnd() % 2 == 0, cumulative = rnd() % 2 == 0;
    Buf kc((size_t)blocks * bs * krow, !odd), vc((size_t)blocks * bs * vrow, !odd);
    std::vector<int32_t> tables((size_t)batch * cols), lens(batch), cu(batch + 1), starts(batch), ws(batch + 1);
    for (auto &t : tables) {
        t = rnd() % 10 == 0 ? (rnd() % 2 ? -1 : blocks + 2) : rnd_in(0, blocks - 1);
    }
    int64_t total = 0;
    cu[0] = 0;
    for (int i = 0; i < batch; ++i) {
        lens[i] = rnd() % 6 == 0 ? 0 : rnd_in(1, bs * cols + bs); // may run past the table: must be skipped
        starts[i] = rnd_in(0, cols + 1) * bs + rnd_in(0, bs - 1);  // may point past the table too
        total += lens[i];
        cu[i + 1] = (int32_t)total;
    }
    // the caller's output may be shorter than the lengths ask for: rows past it must not be written
    const int64_t out_rows = rnd() % 4 == 0 ? total / 2 : total;
    Buf key((size_t)out_rows * krow, !odd), value((size_t)out_rows * vrow, !odd);
    std::vector<uint8_t> kref(key.p, key.p + key.n), vref(value.p, value.p + value.n);
    for (int i = 0; i < batch; ++i) {
        const int64_t start = cu[i];
        for (int t = 0; t * bs < lens[i]; ++t) {
            const int64_t ntok = lens[i] - t * bs < bs ? lens[i] - t * bs : bs;
            const int64_t col = t + (has_starts ? starts[i] / bs : 0);
            if (col >= cols) {
                continue;
            }
            const int64_t blk = tables[(size_t)i * cols + col], row0 = start + (int64_t)t * bs;
            if (blk < 0 || blk >= blocks || row0 + ntok > out_rows) {
                continue;
            }
            std::memcpy(&kref[row0 * krow], kc.p + blk * bs * krow, ntok * krow);
            if (has_v) {
                std::memcpy(&vref[row0 * vrow], vc.p + blk * bs * vrow, ntok * vrow);
            }
        }
    }
    PagedCacheLoadArgs a{};
    a.k_cache = kc.p;
    a.v_cache = has_v ? vc.p : nullptr;
    a.block_tables = tables.data();
    if (cumulative) {
        a.cu_lens = cu.data();
    } else {
        prefix_lens_body(lens.data(), ws.data(), batch);
        a.cu_lens = ws.data();
    }
    a.seq_starts = has_starts ? starts.data() : nullptr;
    a.key = key.p;
    a.value = has_v ? value.p : nullptr;
    a.batch = batch;
    a.table_cols = cols;
    a.block_size = bs;
    a.k_row_bytes = krow;
    a.v_row_bytes = has_v ? vrow : 0;
    a.num_blocks = blocks;
    a.out_rows = out_rows;
    a.chunks = rnd_in(1, 4);
    a.vec16 = !odd && krow % 16 == 0 && a.v_row_bytes % 16 == 0;
    const int threads = rnd_in(1, 5);
    for (int64_t cta = 0; cta < (int64_t)batch * cols * a.chunks; ++cta) {
        for (int tid = 0; tid < threads; ++tid) {
            paged_cache_load_body(a, cta, tid, threads);
        }
    }
    expect(key.n == 0 || std::memcmp(key.p, kref.data(), key.n) == 0, "paged_cache_load key", case_id);
    expect(value.n == 0 || std::memcmp(value.p, vref.data(), value.n) == 0, "paged_cache_load value", case_id);
}

void test_rac_strided(int case_id)
{
    const int tokens = rnd_in(1, 12), slots = rnd_in(1, 40);
    const bool odd = rnd() % 4 == 0, has_v = rnd() % 5 != 0;
    const int64_t krow = odd ? rnd_in(1, 90) : 16 * rnd_in(1, 10), vrow = odd ? rnd_in(1, 90) : 16 * rnd_in(1, 10);
    // rows may overlap (stride < row) or be far apart; the storage holds exactly the last row's end
    const int64_t kstride = odd ? rnd_in(0, 200) : 16 * rnd_in(0, 20), vstride = odd ? rnd_in(0, 200) : 16 * rnd_in(0, 20);
    Buf ks((size_t)((tokens - 1) * kstride + krow), !odd), vs((size_t)((tokens - 1) * vstride + vrow), !odd);
    Buf kc((size_t)slots * krow, !odd), vc((size_t)slots * vrow, !odd);
    std::vector<int32_t> map(tokens);
    std::vector<int> used(slots, 0);
    for (int t = 0; t < tokens; ++t) {
        const uint32_t r = rnd() % 8;
        if (r == 0) {
            map[t] = -1 - (int)(rnd() % 3);
        } else if (r == 1) {
            map[t] = slots + (int)(rnd() % 3);
        } else {
            int sidx = rnd_in(0, slots - 1);
            while (used[sidx]) { // distinct slots, as a block manager hands them out
                sidx = (sidx + 1) % slots;
                if (sidx == 0 && tokens > slots) {
                    break;
                }
            }
            if (used[sidx]) {
                map[t] = -1;
            } else {
                used[sidx] = 1;
                map[t] = sidx;
            }
        }
    }
    std::vector<uint8_t> kref(kc.p, kc.p + kc.n), vref(vc.p, vc.p + vc.n);
    for (int t = 0; t < tokens; ++t) {
        if (map[t] < 0 || map[t] >= slots) {
            continue;
        }
        std::memcpy(&kref[(size_t)map[t] * krow], ks.p + t * kstride, krow);
        if (has_v) {
            std::memcpy(&vref[(size_t)map[t] * vrow], vs.p + t * vstride, vrow);
        }
    }
    RacStridedArgs a{};
    a.key = ks.p;
    a.value = has_v ? vs.p : nullptr;
    a.key_cache = kc.p;
    a.value_cache = has_v ? vc.p : nullptr;
    a.slot_mapping = map.data();
    a.num_tokens = tokens;
    a.k_row_bytes = krow;
    a.v_row_bytes = has_v ? vrow : 0;
    a.k_src_stride = kstride;
    a.v_src_stride = has_v ? vstride : 0;
    a.num_slots = slots;
    a.chunks = rnd_in(1, 4);
    a.vec16 = !odd;
    const int threads = rnd_in(1, 6);
    for (int64_t cta = 0; cta < (int64_t)tokens * a.chunks; ++cta) {
        for (int tid = 0; tid < threads; ++tid) {
            rac_strided_body(a, cta, tid, threads);
        }
    }
    expect(std::memcmp(kc.p, kref.data(), kc.n) == 0, "rac_strided key cache", case_id);
    expect(std::memcmp(vc.p, vref.data(), vc.n) == 0, "rac_strided value cache", case_id);
}

void test_kv_cache(int case_id)
{
    const int layers = rnd_in(1, 3), batch = rnd_in(1, 6), max_seqlen = rnd_in(1, 20);
    const bool odd = rnd() % 4 == 0;
    const int64_t row = odd ? rnd_in(1, 70) : 16 * rnd_in(1, 6);
    std::vector<int32_t> len(batch), off(batch);
    int64_t tokens = 0;
    for (int b = 0; b < batch; ++b) {
        const uint32_t r = rnd() % 10;
        len[b] = r == 0 ? -1 : (r == 1 ? 0 : rnd_in(1, max_seqlen));
        off[b] = r == 2 ? len[b] - 1 : (r == 3 ? max_seqlen + 1 : rnd_in(len[b] > 0 ? len[b] : 0, max_seqlen));
        tokens += len[b] > 0 ? len[b] : 0;
    }
    const bool short_input = rnd() % 6 == 0 && tokens > 1; // new_kv holds fewer rows than the lengths add up to
    const int64_t have = short_input ? tokens - 1 : tokens;
    int32_t layer = (rnd() % 8 == 0) ? layers : rnd_in(0, layers - 1); // sometimes past the cache
    Buf kv((size_t)(have > 0 ? have : 1) * row, !odd), past((size_t)layers * batch * max_seqlen * row, !odd);
    std::vector<uint8_t> ref(past.p, past.p + past.n);
    int64_t prefix = 0;
    for (int b = 0; b < batch; ++b) {
        const int64_t n = len[b];
        if (layer < layers && n > 0 && off[b] >= n && off[b] <= max_seqlen && prefix + n <= have) {
            std::memcpy(&ref[(size_t)(((int64_t)layer * batch + b) * max_seqlen + off[b] - n) * row], kv.p + prefix * row,
                        (size_t)(n * row));
        }
        prefix += n > 0 ? n : 0;
    }
    KvCacheArgs a{};
    a.new_kv = kv.p;
    a.past = past.p;
    a.layer_id = &layer;
    a.token_offset = off.data();
    a.seq_len = len.data();
    a.layers = layers;
    a.batch = batch;
    a.max_seqlen = max_seqlen;
    a.row_bytes = row;
    a.n_tokens = have;
    a.chunks = rnd_in(1, 4);
    a.vec16 = !odd;
    const int threads = rnd_in(1, 6);
    for (int64_t cta = 0; cta < (int64_t)batch * a.chunks; ++cta) {
        for (int tid = 0; tid < threads; ++tid) {
            kv_cache_body(a, cta, tid, threads);
        }
    }
    expect(std::memcmp(past.p, ref.data(), past.n) == 0, "kv_cache past", case_id);
}

} // namespace

int main(int argc, char **argv)
{
    const int n = argc > 1 ? std::atoi(argv[1]) : 400;
    for (int i = 0; i < n; ++i) {
        test_block_copy(i);
        test_paged_cache_load(i);
        test_rac_strided(i);
        test_kv_cache(i);
    }
    std::printf("%d cases, %d failures\n", 4 * n, failures);
    return failures == 0 ? 0 : 1;
}
