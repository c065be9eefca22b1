// Host code: fills the descriptors of one step - token ids, positions, the entry of every token, first token row and
// cached length of every entry, wanted rows, state slots, block tables, and the places of tokens that are still on the
// device - into one pinned buffer that goes to the device in a single copy. This is the per-step work InfiniLM does in
// csrc/engine/infer_engine.cpp:187-254 (batch -> device tensors) from what
// python/infinilm/processors/basic_llm_processor.py:161-263 flattens; done entry by entry in Python it cost the host
// more per step than the GPU needed to run a step of a few hundred requests.
//
// Entries are given in the caller's order (arrays indexed by caller index i); `order[k]` is the caller index of the
// entry that runs k-th (single tokens first). Layout of `out` (int32), in this order; offsets[w] receives where part w
// starts and offsets[11] the total:
//   0 tok[Tp]  1 pos[Tp]  2 ent[Tp]  3 qstart[Ep+1]  4 kvlen[Ep]  5 want[max(n_want,1)]  6 read_slot[Ep]  7 write_slot[Ep]
//   8 block tables, group after group, each [Ep][width[g]]  9 patch_row[n_patch_cap]  10 patch_src[n_patch_cap]
// A token given as -(1 + s) is not known to the host: its row and s go to the patch lists and the device fills it in.
// A step that is replayed as a graph has Ep - E padding entries behind its first `pad_at` entries (the single tokens):
// one token each at position 0 of the scratch page, state from the zero slot into the scratch slot. Its list of wanted
// rows has a fixed length n_want_fixed: the rows asked for, in the caller's order, then row 0 again and again.
// Returns 0, or a negative code with *bad_entry = the caller index at fault:
//   -11 a wanted place outside the entry's tokens, -12 a block table longer than its group's width,
//   -13 `out` too small, -14 more device tokens than patch room, -15 counts that do not fit together.
#include <cstdint>
#include <cstring>

extern "C" __attribute__((visibility("default")))
int il_step_fill(int32_t* out, long long out_cap, int E, int Ep, int Tp, const int32_t* order, const int32_t* n_tok,
                 const int32_t* start, const int32_t* slot, const uint8_t* fresh, const long long* tokens,
                 const int32_t* tok_off, int n_groups, const int32_t* widths, const unsigned long long* tbl_ptr,
                 const int32_t* tbl_len, const int32_t* scratch_page, int scratch_slot, const int32_t* want,
                 const int32_t* want_off, int pad_at, int n_want_fixed, int n_patch_cap, int32_t* offsets,
                 int32_t* n_patch_out, int32_t* n_want_out, int32_t* bad_entry) {
    *bad_entry = -1;
    const int n_pad = Ep - E;
    const bool graph_mode = n_want_fixed >= 0;
    if (n_pad < 0 || pad_at < 0 || pad_at > E || (n_pad > 0 && !graph_mode) || (graph_mode && want_off[E] > n_want_fixed)) return -15;
    const long long n_want = graph_mode ? n_want_fixed : want_off[E];
    long long off = 0;
    auto take = [&](int which, long long n) {
        offsets[which] = (int32_t)off;
        off += n;
    };
    take(0, Tp), take(1, Tp), take(2, Tp), take(3, Ep + 1), take(4, Ep), take(5, n_want > 0 ? n_want : 1), take(6, Ep), take(7, Ep);
    offsets[8] = (int32_t)off;
    for (int g = 0; g < n_groups; ++g) off += (long long)Ep * widths[g];
    take(9, n_patch_cap), take(10, n_patch_cap);
    offsets[11] = (int32_t)off;
    *n_want_out = (int32_t)n_want;
    if (off > out_cap) return -13;
    int32_t *tok = out + offsets[0], *pos = out + offsets[1], *ent = out + offsets[2], *qs = out + offsets[3];
    int32_t *kv = out + offsets[4], *wr = out + offsets[5], *rs = out + offsets[6], *wsl = out + offsets[7];
    int32_t *prow = out + offsets[9], *psrc = out + offsets[10];

    // rows in running order; tokens, positions, entries, device tokens
    int n_patch = 0;
    qs[0] = 0;
    for (int k = 0; k < Ep; ++k) {
        const int a = qs[k];
        if (k >= pad_at && k < pad_at + n_pad) {  // a padding entry
            tok[a] = 0, pos[a] = 0, ent[a] = k;
            qs[k + 1] = a + 1;
            kv[k] = 1, rs[k] = 0, wsl[k] = scratch_slot;
            continue;
        }
        const int i = order[k < pad_at ? k : k - n_pad], n = n_tok[i], s = start[i];
        const long long* src = tokens + tok_off[i];
        for (int j = 0; j < n; ++j) {
            const long long t = src[j];
            if (t < 0) {
                if (n_patch >= n_patch_cap) {
                    *bad_entry = i;
                    return -14;
                }
                prow[n_patch] = a + j;
                psrc[n_patch++] = (int32_t)(-1 - t);
                tok[a + j] = 0;
            } else {
                tok[a + j] = (int32_t)t;
            }
            pos[a + j] = s + j;
            ent[a + j] = k;
        }
        qs[k + 1] = a + n;
        kv[k] = s + n;
        rs[k] = fresh[i] ? 0 : slot[i];
        wsl[k] = slot[i];
    }
    if (qs[Ep] != Tp) return -15;
    // wanted rows: the flat list `want` is in the caller's order, and so are the rows that come out (place j stays place j)
    for (int k = 0; k < Ep; ++k) {
        if (k >= pad_at && k < pad_at + n_pad) continue;
        const int i = order[k < pad_at ? k : k - n_pad], base = qs[k], n = n_tok[i];
        for (int j = want_off[i]; j < want_off[i + 1]; ++j) {
            const int w = want[j];
            if (w < 0 || w >= n) {
                *bad_entry = i;
                return -11;
            }
            wr[j] = base + w;
        }
    }
    for (long long j = want_off[E]; j < n_want; ++j) wr[j] = 0;
    // block tables: a row per entry, -1 behind its pages; padding rows write to the scratch page
    long long g_off = offsets[8];
    for (int g = 0; g < n_groups; ++g) {
        const int w = widths[g];
        int32_t* bt = out + g_off;
        for (int k = 0; k < Ep; ++k) {
            int32_t* row = bt + (long long)k * w;
            if (k >= pad_at && k < pad_at + n_pad) {
                for (int j = 1; j < w; ++j) row[j] = -1;
                row[0] = scratch_page[g];
                continue;
            }
            const int i = order[k < pad_at ? k : k - n_pad];
            const int len = tbl_len[(long long)g * E + i];
            if (len > w) {
                *bad_entry = i;
                return -12;
            }
            if (len > 0) memcpy(row, reinterpret_cast<const int32_t*>((uintptr_t)tbl_ptr[(long long)g * E + i]), (size_t)len * 4);
            for (int j = len; j < w; ++j) row[j] = -1;
        }
        g_off += (long long)Ep * w;
    }
    *n_patch_out = n_patch;
    return 0;
}
