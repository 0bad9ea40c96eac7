// Host-side GEMM front-end: GemmConfig presets, names, grids, kernarg blobs, auto_select and the mapping of a
// GemmConfig onto the sm_100a kernel family.  Mirrors the public functions of src/t0/gemm_gen.rs (reference
// project paths); the RDNA3 code generator behind them is replaced by precompiled tcgen05 kernels.
#include <sys/stat.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <mutex>
#include <string>
#include <unordered_map>

#include "t0b_internal.hpp"

namespace {

t0b_gemm_config make_cfg(uint32_t tm, uint32_t tn, uint32_t tk, uint32_t wg, bool lds, bool db, uint32_t passes = 1) {
    t0b_gemm_config c{};
    c.tile_m = tm;
    c.tile_n = tn;
    c.tile_k = tk;
    c.wg_size = wg;
    c.use_lds = lds;
    c.double_buffer = db;
    c.split_k = 0;
    c.lds_pad = 0;
    c.n_col_passes = passes;
    c.swap_grid = 1;
    c.wgp_mode = 1;
    c.transpose = T0B_TRANSPOSE_NT;
    c.epilogue = T0B_EPI_STORE_F32;
    return c;
}

struct Preset {
    const char* name;
    t0b_gemm_config cfg;
};

// The reference's presets (gemm_gen.rs:86-145) followed by the B200-native tiles.
const Preset* presets(int* count) {
    static const Preset table[] = {
        {"16x64_k16", make_cfg(16, 64, 16, 32, true, true)},
        {"32x64_direct", make_cfg(32, 64, 16, 64, false, false)},
        {"32x64_k16", make_cfg(32, 64, 16, 64, true, true)},
        {"32x64_k32", make_cfg(32, 64, 32, 64, true, true)},
        {"32x128_k16", make_cfg(32, 128, 16, 64, true, true)},
        {"64x64_k16", make_cfg(64, 64, 16, 64, true, true)},
        {"64x64_k32", make_cfg(64, 64, 32, 64, true, true)},
        {"128x64_k16", make_cfg(128, 64, 16, 128, true, true)},
        {"64x128_k16", make_cfg(64, 128, 16, 64, true, true)},
        {"128x64_k32", make_cfg(128, 64, 32, 128, true, true)},
        {"128x128_k16", make_cfg(128, 128, 16, 128, true, true)},
        {"64x64_k64", make_cfg(64, 64, 64, 64, true, true)},
        {"128x128_2pass", make_cfg(128, 64, 16, 128, true, true, 2)},
        {"64x128_2pass", make_cfg(64, 64, 16, 64, true, true, 2)},
        {"b200_128x64", make_cfg(128, 64, 64, 192, true, true)},
        {"b200_128x128", make_cfg(128, 128, 64, 192, true, true)},
        {"b200_128x256", make_cfg(128, 256, 64, 192, true, true)},
        {"b200_256x128", make_cfg(256, 128, 64, 192, true, true)},
        {"b200_256x256", make_cfg(256, 256, 64, 192, true, true)},
        {"b200_512x256", make_cfg(512, 256, 64, 320, true, true)},
        {"b200_256x512", make_cfg(256, 512, 64, 320, true, true)},
    };
    *count = static_cast<int>(sizeof(table) / sizeof(table[0]));
    return table;
}

t0b_gemm_config preset_or_die(const char* name) {
    int n;
    const Preset* t = presets(&n);
    for (int i = 0; i < n; ++i)
        if (std::strcmp(t[i].name, name) == 0) return t[i].cfg;
    return make_cfg(64, 64, 16, 64, true, true);
}

uint32_t sk_of(const t0b_gemm_config* c) { return c->split_k == 0 ? 1u : c->split_k; }

void put_u64(uint8_t* p, uint64_t v) {
    for (int i = 0; i < 8; ++i) p[i] = static_cast<uint8_t>(v >> (8 * i));
}
void put_u32(uint8_t* p, uint32_t v) {
    for (int i = 0; i < 4; ++i) p[i] = static_cast<uint8_t>(v >> (8 * i));
}

int stage_bytes(uint32_t bn, uint32_t cg, uint32_t mt) {
    return static_cast<int>(mt) * 128 * 64 * 2 + static_cast<int>(bn / cg) * 64 * 2;
}

// Epilogue warps of a variant: four per accumulator owner, doubled for single-accumulator tiles of >= 128 columns.
int epi_warps(uint32_t bn, uint32_t mt) { return static_cast<int>(mt) * 4 * ((mt == 1 && bn >= 128) ? 2 : 1); }

int stages_for(uint32_t bn, uint32_t cg, uint32_t mt) {
    const int stage = stage_bytes(bn, cg, mt);
    const int budget = 227 * 1024 - 1024 - 1024 - epi_warps(bn, mt) * 4096;   // minus the epilogue transpose tiles
    return std::min(8, budget / stage);
}

}  // namespace

namespace t0b {

// ---- measured configs: this process's tuner results, then the shipped table ------------------------------------
struct TunedRow {
    uint32_t m, n, k;
    int trans_a, trans_b, out_bf16;
    const char* tile;          // preset name
    uint32_t split_k, swap_grid, group;   // group: rasterisation group width (0 = automatic), carried in lds_pad
    float tflops;
};
// Measured on B200 with t0b_tune (python -m t0_gpu_b200.make_tuned_table), one row per benchmark shape and layout.
static const TunedRow kShippedTable[] = {
#include "t0b_tuned_table.inc"
};

static std::mutex g_tuned_mu;
static std::unordered_map<std::string, t0b_gemm_config>& process_tuned() {
    static std::unordered_map<std::string, t0b_gemm_config> map;
    return map;
}

std::string tuned_key(uint32_t m, uint32_t n, uint32_t k, int trans_a, int trans_b, int out_bf16) {
    return std::to_string(m) + "x" + std::to_string(n) + "x" + std::to_string(k) + "/" + std::to_string(trans_a != 0) +
           std::to_string(trans_b != 0) + std::to_string(out_bf16 != 0);
}

void tuned_remember(uint32_t m, uint32_t n, uint32_t k, int trans_a, int trans_b, int out_bf16, const t0b_gemm_config& cfg) {
    std::lock_guard<std::mutex> lk(g_tuned_mu);
    process_tuned()[tuned_key(m, n, k, trans_a, trans_b, out_bf16)] = cfg;
}

void tuned_forget(uint32_t m, uint32_t n, uint32_t k) {
    std::lock_guard<std::mutex> lk(g_tuned_mu);
    for (int bits = 0; bits < 8; ++bits) process_tuned().erase(tuned_key(m, n, k, bits & 4, bits & 2, bits & 1));
}

// source: 2 = measured in this process, 1 = the shipped table.
bool tuned_lookup(uint32_t m, uint32_t n, uint32_t k, int trans_a, int trans_b, int out_bf16, t0b_gemm_config* out, int* source) {
    {
        std::lock_guard<std::mutex> lk(g_tuned_mu);
        auto it = process_tuned().find(tuned_key(m, n, k, trans_a, trans_b, out_bf16));
        if (it != process_tuned().end()) {
            *out = it->second;
            if (source) *source = 2;
            return true;
        }
    }
    for (const TunedRow& r : kShippedTable) {
        if (r.m != m || r.n != n || r.k != k || (r.trans_a != 0) != (trans_a != 0) || (r.trans_b != 0) != (trans_b != 0) ||
            (r.out_bf16 != 0) != (out_bf16 != 0))
            continue;
        if (t0b_config_preset(r.tile, out) != T0B_OK) continue;
        out->split_k = r.split_k > 1 ? r.split_k : 0;
        out->swap_grid = r.swap_grid;
        out->lds_pad = r.group;
        if (source) *source = 1;
        return true;
    }
    return false;
}

// Pick the B200 tile for a shape with a small cost model whose constants were measured on B200 (on-device tuner,
// random operands, SM clock ~1.5 GHz under tensor load).  It stands where the reference has its RDNA3 cost model
// (src/t0/cost_model.rs:168-471): estimate the time of every candidate, keep the cheapest.
//   time = waves * (k_blocks * cycles_per_k_block + exposed_epilogue) + launch, plus the slab reduce for split-K.
// cycles_per_k_block: measured with in-kernel timer stamps (the timeline build).  Shared-memory bandwidth bounds the
// main loop: the two-accumulator tiles (256x512, 512x256) need 128 B/clk and run 8 MMAs in ~1165 cycles, the 256x256
// pair tile needs 160 B/clk (4 MMAs in ~780), the 128x256 single-CTA tile 192 B/clk (4 MMAs in ~760); narrower MMAs
// take the same time for fewer columns.  The two-accumulator tiles cannot hide their epilogue.  The exchange of a
// cluster split-K (barrier, sum over distributed shared memory, closing barrier) costs ~7000 cycles.
void default_b200_config(uint32_t m, uint32_t k, uint32_t n, int num_sms, t0b_gemm_config* out) {
    struct Cand {
        uint32_t bm, bn, cg;
        double kb_cycles;      // per 64-deep K block, per CTA
        double epi_exposed;    // cycles per tile the MMA pipe idles for the epilogue
        double epi_tail;       // cycles after the last tile
    };
    static const Cand cands[] = {
        {256, 512, 2, 1165.0, 10000.0, 0.0}, {512, 256, 2, 1175.0, 10000.0, 0.0}, {256, 256, 2, 780.0, 0.0, 8000.0},
        {128, 256, 1, 760.0, 0.0, 8000.0},   {128, 128, 1, 700.0, 0.0, 5000.0},   {128, 64, 1, 550.0, 0.0, 3500.0},
    };
    if (num_sms <= 0) num_sms = 148;
    const uint32_t kb_total = std::max(1u, (k + 63) / 64);
    double best = 1e300;
    Cand pick = cands[4];
    uint32_t pick_sk = 1;
    for (const Cand& c : cands) {
        const uint64_t tiles = static_cast<uint64_t>((m + c.bm - 1) / c.bm) * ((n + c.bn - 1) / c.bn);
        const uint64_t clusters = static_cast<uint64_t>(num_sms) / c.cg;
        for (uint32_t sk = 1; sk <= 16; sk *= 2) {
            if (sk > 1 && (kb_total / sk < 4 || tiles * (sk / 2) >= clusters)) break;   // split only while the grid is not full
            const uint32_t kbps = (kb_total + sk - 1) / sk;
            const uint64_t work = tiles * sk;
            const uint64_t waves = (work + clusters - 1) / clusters;
            double cyc = static_cast<double>(waves) * (kbps * c.kb_cycles + c.epi_exposed) + c.epi_tail + 4500.0;
            // The hidden epilogue of a double-buffered tile still bounds a tile whose main loop is shorter than it.
            if (c.epi_exposed == 0.0 && kbps * c.kb_cycles < c.epi_tail) cyc += static_cast<double>(waves - 1) * (c.epi_tail - kbps * c.kb_cycles);
            if (sk > 1) {
                // Single-CTA tiles with up to four K ranges (eight when all clusters fit at once: GPC sizes allow about
                // fifteen eight-CTA clusters) sum their partials inside a thread-block cluster (~7000 cycles: barrier, sum
                // over distributed shared memory, closing barrier); the rest pay the slab round trip and a second kernel
                // (measured ~6 us more than the cluster path on 128x4096x4096: launch hand-over + bytes at ~5 TB/s).
                const bool in_cluster = c.cg == 1 && (sk <= 4 || (sk == 8 && tiles <= 15));
                cyc += in_cluster ? 7000.0 : 14000.0 + static_cast<double>(m) * n * 4.0 * (sk + 1) / 3300.0;
            }
            if (cyc < best) {
                best = cyc;
                pick = c;
                pick_sk = sk;
            }
        }
    }
    t0b_gemm_config cfg = make_cfg(pick.bm, pick.bn, 64, (pick.bm >= 512 || pick.bn >= 512) ? 320 : 192, true, true);
    cfg.wgp_mode = pick.cg == 2;
    cfg.swap_grid = (m >= n) ? 1 : 0;
    cfg.split_k = pick_sk > 1 ? pick_sk : 0;
    *out = cfg;
}

void resolve_plan(const t0b_gemm_config* cfg_in, const PlanInput& in, t0b_gemm_plan* out) {
    t0b_gemm_config cfg;
    if (cfg_in) cfg = *cfg_in;
    else default_b200_config(in.m, in.k, in.n, in.num_sms, &cfg);
    const int num_sms = in.num_sms > 0 ? in.num_sms : 148;
    t0b_gemm_plan p{};
    p.cta_group = cfg.tile_m >= 256 ? 2 : 1;
    const uint32_t want_n = cfg.tile_n * std::max(1u, cfg.n_col_passes);
    p.bn = want_n <= 64 ? 64 : (want_n <= 128 ? 128 : 256);
    if (p.cta_group == 2 && p.bn < 128) p.bn = 128;
    // Both TMEM accumulators in one tile: two N-adjacent 256-wide halves sharing A (tile_n >= 512, CTA pair), or two
    // M-adjacent halves sharing B (tile_m >= 512).
    p.n_tiles = (want_n >= 512 && p.cta_group == 2) ? 2 : 1;
    p.m_tiles = (p.n_tiles == 1 && cfg.tile_m >= 512 && p.bn == 256) ? 2 : 1;
    if (p.n_tiles == 2) p.bn = 512;
    p.bm = 128 * p.cta_group * p.m_tiles;
    p.bk = 64;
    p.stages = static_cast<uint32_t>(stages_for(p.n_tiles == 2 ? 256 : p.bn, p.cta_group, std::max(p.m_tiles, p.n_tiles)));
    const uint32_t kb_total = (in.k + 63) / 64;
    uint32_t sk = std::max(1u, sk_of(&cfg));
    sk = std::min(sk, std::max(1u, kb_total));
    const uint32_t kbps = kb_total == 0 ? 0 : (kb_total + sk - 1) / sk;
    p.kb_per_split = kbps;
    p.split_k = kbps == 0 ? 1 : (kb_total + kbps - 1) / kbps;
    p.use_tma = (in.a_ptr % 16 == 0) && (in.b_ptr % 16 == 0) && ((in.lda * 2) % 16 == 0) && ((in.ldb * 2) % 16 == 0) &&
                in.lda > 0 && in.ldb > 0;
    const uint64_t tiles = static_cast<uint64_t>((in.m + p.bm - 1) / p.bm) * ((in.n + p.bn - 1) / p.bn) * p.split_k;
    const uint64_t clusters = static_cast<uint64_t>(num_sms) / p.cta_group;
    p.grid = static_cast<uint32_t>(std::min<uint64_t>(tiles, clusters) * p.cta_group);
    p.smem_bytes = p.stages * stage_bytes(p.n_tiles == 2 ? 256 : p.bn, p.cta_group, std::max(p.m_tiles, p.n_tiles)) + 1024 + 1024 +
                   epi_warps(p.n_tiles == 2 ? 256 : p.bn, std::max(p.m_tiles, p.n_tiles)) * 4096;
    *out = p;
}

}  // namespace t0b

extern "C" {

int32_t t0b_config_preset(const char* name, t0b_gemm_config* out) {
    if (!name || !out) return T0B_ERR_INVALID;
    std::string s(name);
    if (s.rfind("tile_", 0) == 0) s = s.substr(5);
    int n;
    const Preset* t = presets(&n);
    for (int i = 0; i < n; ++i)
        if (s == t[i].name) {
            *out = t[i].cfg;
            return T0B_OK;
        }
    return T0B_ERR_INVALID;
}

int32_t t0b_config_name(const t0b_gemm_config* c, char* buf, size_t cap) {
    if (!c || !buf || cap == 0) return T0B_ERR_INVALID;
    std::string s = "t0_gemm_" + std::to_string(c->tile_m) + "x" + std::to_string(c->tile_n) + "_k" +
                    std::to_string(c->tile_k);
    s += c->use_lds ? (c->double_buffer ? "_ldsdb" : "_lds") : "_direct";
    if (c->split_k > 1) s += "_sk" + std::to_string(c->split_k);
    if (c->n_col_passes > 1) s += "_" + std::to_string(c->n_col_passes) + "p";
    if (!c->swap_grid) s += "_mg";
    if (c->wgp_mode) s += "_wgp";
    if (c->transpose == T0B_TRANSPOSE_NN) s += "_nn";
    if (c->epilogue == T0B_EPI_BIAS_ADD) s += "_bias";
    else if (c->epilogue == T0B_EPI_BIAS_ADD_RELU) s += "_bias_relu";
    const size_t len = std::min(s.size(), cap - 1);
    std::memcpy(buf, s.data(), len);
    buf[len] = 0;
    return static_cast<int32_t>(len);
}

int32_t t0b_sweep_configs(t0b_gemm_config* out, int32_t cap) {
    static const char* names[] = {"16x64_k16", "32x64_k16",  "32x64_k32",  "32x128_k16", "64x64_k16",
                                  "64x64_k32", "128x64_k16", "64x128_k16", "128x64_k32"};
    const int32_t n = 9;
    for (int32_t i = 0; i < n && i < cap && out; ++i) out[i] = preset_or_die(names[i]);
    return n;
}

int32_t t0b_standard_configs(t0b_gemm_config* out, int32_t cap) {
    struct E {
        const char* name;
        uint32_t sk;
    };
    static const E list[] = {{"16x64_k16", 0},  {"32x64_k16", 0}, {"32x64_k32", 0}, {"32x128_k16", 0}, {"64x64_k16", 0},
                             {"64x64_k32", 0},  {"128x64_k32", 0}, {"32x64_k32", 2}, {"16x64_k16", 4},  {"64x64_k32", 2},
                             {"64x64_k16", 4},  {"64x64_k32", 4},  {"64x64_k16", 8}, {"128x64_k32", 2}};
    const int32_t n = 14;
    for (int32_t i = 0; i < n && i < cap && out; ++i) {
        out[i] = preset_or_die(list[i].name);
        out[i].split_k = list[i].sk;
    }
    return n;
}

uint32_t t0b_config_lds_total(const t0b_gemm_config* c) {
    if (!c) return 0;
    const uint32_t per = c->tile_m * c->tile_k * 2 + c->tile_n * c->tile_k * 2;
    return c->double_buffer ? per * 2 : per;
}

uint32_t t0b_config_estimated_vgprs(const t0b_gemm_config* c) {
    if (!c || c->wg_size < 32) return 0;
    const uint32_t n_waves = c->wg_size / 32;
    const uint32_t nrb = (c->tile_m / n_waves) / 16;
    const uint32_t nct = c->tile_n / 16;
    const uint32_t x_lpt = (c->tile_m * c->tile_k * 2 / c->wg_size) / 16;
    const uint32_t wt_lpt = (c->tile_n * c->tile_k * 2 / c->wg_size) / 16;
    return nrb * nct * 8 + nrb * 8 + nct * 8 + x_lpt * 4 + wt_lpt * 4 + 49;
}

// The reference rejects configs whose RDNA3 register estimate exceeds 256 (gemm_gen.rs:189-205).  On B200 the
// accumulators live in TMEM, so every config that maps onto the kernel family is feasible.
int32_t t0b_config_is_feasible(const t0b_gemm_config* c) {
    if (!c) return 0;
    return c->tile_m >= 1 && c->tile_n >= 1 && c->tile_k >= 1 && (c->split_k == 0 || (c->split_k & (c->split_k - 1)) == 0);
}

int32_t t0b_auto_select(uint32_t m, uint32_t k, uint32_t n, t0b_gemm_config* out) {
    if (!out || m == 0 || n == 0 || k == 0) return T0B_ERR_INVALID;
    // Like the reference's predict_best over its tune cache (src/t0/cost_model.rs:593-601, 788-1078): a measurement of
    // this process first, then the table measured on B200 that ships with the library, then the cost model.  The
    // call carries no layout, so the NT / f32 entry (the reference's only layout) is preferred, then NN, then any.
    static const int order[][3] = {{0, 1, 0}, {0, 0, 0}, {1, 0, 0}, {1, 1, 0}, {0, 1, 1}, {0, 0, 1}, {1, 0, 1}, {1, 1, 1}};
    for (const auto& o : order)
        if (t0b::tuned_lookup(m, n, k, o[0], o[1], o[2], out, nullptr)) return T0B_OK;
    t0b::default_b200_config(m, k, n, 148, out);
    return T0B_OK;
}

int32_t t0b_auto_select_source(uint32_t m, uint32_t k, uint32_t n, int32_t trans_a, int32_t trans_b, int32_t out_dtype,
                               t0b_gemm_config* out) {
    if (!out || m == 0 || n == 0 || k == 0) return T0B_ERR_INVALID;
    int source = 0;
    if (t0b::tuned_lookup(m, n, k, trans_a != 0, trans_b != 0, out_dtype == T0B_OUT_BF16, out, &source)) return source;
    t0b::default_b200_config(m, k, n, 148, out);
    return 0;
}

int32_t t0b_auto_select_legacy(uint32_t m, uint32_t k, uint32_t n, t0b_gemm_config* out) {
    if (!out || m == 0 || n == 0 || k == 0) return T0B_ERR_INVALID;
    const uint64_t mn = static_cast<uint64_t>(m) * n;
    // Largest power-of-two split <= desired that keeps K a multiple of tile_k * split.
    auto clamp_sk = [k](uint32_t tile_k, uint32_t desired) -> uint32_t {
        uint32_t sk = std::min(desired, k / tile_k);
        while (sk > 1 && k % (tile_k * sk) != 0) sk /= 2;
        return sk > 1 ? sk : 0;
    };
    const bool m128 = (m % 128 == 0) && m >= 128;
    const bool m64 = (m % 64 == 0);
    const bool wide = k >= 512 && n >= 1024 && m128;
    t0b_gemm_config c;
    if (m <= 256 && wide) {
        c = preset_or_die("128x64_k16"); c.swap_grid = 0; c.split_k = clamp_sk(16, 4);
    } else if (m <= 512 && wide) {
        c = preset_or_die("128x64_k16"); c.swap_grid = 0; c.split_k = clamp_sk(16, 8);
    } else if (mn <= 512ull * 512ull) {
        c = preset_or_die("64x64_k16"); c.swap_grid = 0; c.split_k = clamp_sk(16, 8);
    } else if (mn <= 1024ull * 1024ull && m128) {
        c = preset_or_die("128x64_k16"); c.swap_grid = 0; c.split_k = clamp_sk(16, 2);
    } else if (m128) {
        c = preset_or_die("128x64_k16"); c.split_k = clamp_sk(16, 8);
    } else if (m64) {
        c = preset_or_die("64x64_k16"); c.split_k = clamp_sk(16, 4);
    } else {
        c = preset_or_die("32x64_k16"); c.split_k = clamp_sk(16, 4);
    }
    *out = c;
    return T0B_OK;
}

int32_t t0b_auto_select_backward_data(uint32_t m, uint32_t n_orig, uint32_t k_orig, t0b_gemm_config* out) {
    return t0b_auto_select(m, n_orig, k_orig, out);   // dX[M,K] = dY[M,N] * W: contraction over N_orig
}
int32_t t0b_auto_select_backward_weight(uint32_t m, uint32_t n_orig, uint32_t k_orig, t0b_gemm_config* out) {
    return t0b_auto_select(n_orig, m, k_orig, out);   // dW[N,K] = dY^T * X: contraction over M
}

int32_t t0b_compute_grid(const t0b_gemm_config* c, uint32_t m, uint32_t n, uint32_t* gx, uint32_t* gy) {
    if (!c || !gx || !gy || c->tile_m == 0 || c->tile_n == 0) return T0B_ERR_INVALID;
    const uint32_t eff_n = c->tile_n * std::max(1u, c->n_col_passes);
    const uint32_t tiles_m = (m + c->tile_m - 1) / c->tile_m;
    const uint32_t tiles_n = (n + eff_n - 1) / eff_n;
    if (c->swap_grid) { *gx = tiles_n * c->wg_size; *gy = tiles_m; }
    else { *gx = tiles_m * c->wg_size; *gy = tiles_n; }
    return T0B_OK;
}

int32_t t0b_compute_grid_split_k(const t0b_gemm_config* c, uint32_t m, uint32_t n, uint32_t sk, uint32_t* gx,
                                 uint32_t* gy) {
    if (sk == 0 || (sk & (sk - 1)) != 0) return T0B_ERR_INVALID;   // the reference asserts a power of two
    const int32_t rc = t0b_compute_grid(c, m, n, gx, gy);
    if (rc != T0B_OK) return rc;
    *gy *= sk;
    return T0B_OK;
}

int32_t t0b_compute_grid_auto(const t0b_gemm_config* c, uint32_t m, uint32_t n, uint32_t* gx, uint32_t* gy) {
    if (!c) return T0B_ERR_INVALID;
    const uint32_t sk = sk_of(c);
    return sk > 1 ? t0b_compute_grid_split_k(c, m, n, sk, gx, gy) : t0b_compute_grid(c, m, n, gx, gy);
}

int32_t t0b_compute_grid_backward_data(const t0b_gemm_config* c, uint32_t m, uint32_t k_orig, uint32_t* gx,
                                       uint32_t* gy) {
    return t0b_compute_grid_auto(c, m, k_orig, gx, gy);
}
int32_t t0b_compute_grid_backward_weight(const t0b_gemm_config* c, uint32_t n_orig, uint32_t k_orig, uint32_t* gx,
                                         uint32_t* gy) {
    return t0b_compute_grid_auto(c, n_orig, k_orig, gx, gy);
}

int32_t t0b_build_kernargs(uint64_t x, uint64_t wt, uint64_t y, uint32_t k, uint32_t n, uint32_t m,
                           const t0b_gemm_config* c, uint8_t out[40]) {
    if (!c || !out) return T0B_ERR_INVALID;
    const uint32_t y_stride = sk_of(c) > 1 ? m * n * 4u : 0u;
    put_u64(out + 0, x);
    put_u64(out + 8, wt);
    put_u64(out + 16, y);
    put_u32(out + 24, k);
    put_u32(out + 28, n);
    put_u32(out + 32, 0);
    put_u32(out + 36, y_stride);
    return T0B_OK;
}

int32_t t0b_build_kernargs_with_bias(uint64_t x, uint64_t wt, uint64_t y, uint32_t k, uint32_t n, uint32_t m,
                                     const t0b_gemm_config* c, uint64_t bias, uint8_t out[48]) {
    const int32_t rc = t0b_build_kernargs(x, wt, y, k, n, m, c, out);
    if (rc != T0B_OK) return rc;
    put_u64(out + 40, bias);
    return T0B_OK;
}

int32_t t0b_build_kernargs_m(uint64_t x, uint64_t wt, uint64_t y, uint32_t k, uint32_t n, uint32_t m, uint8_t out[44]) {
    if (!out) return T0B_ERR_INVALID;
    put_u64(out + 0, x);
    put_u64(out + 8, wt);
    put_u64(out + 16, y);
    put_u32(out + 24, k);
    put_u32(out + 28, n);
    put_u32(out + 32, 0);
    put_u32(out + 36, 0);
    put_u32(out + 40, m);
    return T0B_OK;
}

int32_t t0b_build_kernargs_backward_data(uint64_t dy, uint64_t w, uint64_t dx, uint32_t m, uint32_t n_orig,
                                         uint32_t k_orig, const t0b_gemm_config* c, uint8_t out[40]) {
    return t0b_build_kernargs(dy, w, dx, n_orig, k_orig, m, c, out);
}
int32_t t0b_build_kernargs_backward_weight(uint64_t dy_t, uint64_t x_t, uint64_t dw, uint32_t m, uint32_t n_orig,
                                           uint32_t k_orig, const t0b_gemm_config* c, uint8_t out[40]) {
    return t0b_build_kernargs(dy_t, x_t, dw, m, k_orig, n_orig, c, out);
}

int32_t t0b_resolve_plan(const t0b_gemm_config* cfg, uint32_t m, uint32_t n, uint32_t k, int32_t trans_a,
                         int32_t trans_b, uint64_t lda, uint64_t ldb, int32_t num_sms, t0b_gemm_plan* out) {
    if (!out) return T0B_ERR_INVALID;
    t0b::PlanInput in{m, n, k, trans_a, trans_b, lda, ldb, 0, 0, num_sms};
    t0b::resolve_plan(cfg, in, out);
    return T0B_OK;
}

size_t t0b_gemm_workspace_bytes(const t0b_gemm_config* cfg, uint32_t m, uint32_t n, uint32_t k) {
    t0b_gemm_plan p;
    t0b::PlanInput in{m, n, k, 0, 1, k, k, 0, 0, 148};
    t0b::resolve_plan(cfg, in, &p);
    return p.split_k > 1 ? static_cast<size_t>(p.split_k) * m * n * 4 : 0;
}

// ------------------------------------------------------------------------------------------------ autotune cache

static std::string tune_dir(const char* dir) {
    if (dir && *dir) return dir;
    if (const char* e = std::getenv("T0_AUTOTUNE_DIR")) return e;
    const char* home = std::getenv("HOME");
    return std::string(home ? home : ".") + "/.t0_autotune";
}
static std::string tune_path(const char* dir, uint32_t m, uint32_t n, uint32_t k) {
    return tune_dir(dir) + "/gemm_" + std::to_string(m) + "x" + std::to_string(n) + "x" + std::to_string(k) + ".json";
}
// Minimal key lookup in the flat JSON object the cache files hold.
static bool json_number(const std::string& text, const char* key, double* out) {
    const std::string pat = std::string("\"") + key + "\":";
    const size_t at = text.find(pat);
    if (at == std::string::npos) return false;
    const char* p = text.c_str() + at + pat.size();
    char* end = nullptr;
    const double v = std::strtod(p, &end);
    if (end == p) return false;
    *out = v;
    return true;
}

int32_t t0b_tune_cache_save(const char* dir, uint32_t m, uint32_t n, uint32_t k, const t0b_gemm_config* c, float tflops) {
    if (!c) return T0B_ERR_INVALID;
    const std::string d = tune_dir(dir);
    ::mkdir(d.c_str(), 0755);
    char name[160];
    t0b_config_name(c, name, sizeof(name));
    char buf[640];
    std::snprintf(buf, sizeof(buf),
                  "{\"tile_m\":%u,\"tile_n\":%u,\"tile_k\":%u,\"wg_size\":%u,\"split_k\":%u,\"lds_pad\":%u,\"n_col_passes\":%u,"
                  "\"wgp\":%s,\"swap\":%s,\"tflops\":%.2f,\"all\":[[\"%s\",%.2f]]}",
                  c->tile_m, c->tile_n, c->tile_k, c->wg_size, c->split_k > 1 ? c->split_k : 1u, c->lds_pad, c->n_col_passes,
                  c->wgp_mode ? "true" : "false", c->swap_grid ? "true" : "false", tflops, name, tflops);
    std::ofstream f(tune_path(dir, m, n, k));
    if (!f) return T0B_ERR_INVALID;
    f << buf;
    return f.good() ? T0B_OK : T0B_ERR_INVALID;
}

int32_t t0b_tune_cache_load(const char* dir, uint32_t m, uint32_t n, uint32_t k, t0b_gemm_config* c, float* tflops) {
    if (!c) return T0B_ERR_INVALID;
    std::ifstream f(tune_path(dir, m, n, k));
    if (!f) return T0B_ERR_INVALID;
    std::stringstream ss;
    ss << f.rdbuf();
    const std::string text = ss.str();
    double tm, tn, tk, wg, tf, v;
    if (!json_number(text, "tile_m", &tm) || !json_number(text, "tile_n", &tn) || !json_number(text, "tile_k", &tk) ||
        !json_number(text, "wg_size", &wg) || !json_number(text, "tflops", &tf))
        return T0B_ERR_INVALID;
    t0b_gemm_config cfg = make_cfg(static_cast<uint32_t>(tm), static_cast<uint32_t>(tn), static_cast<uint32_t>(tk),
                                   static_cast<uint32_t>(wg), true, true);
    cfg.split_k = (json_number(text, "split_k", &v) && v > 1) ? static_cast<uint32_t>(v) : 0;
    cfg.lds_pad = json_number(text, "lds_pad", &v) ? static_cast<uint32_t>(v) : 0;
    cfg.n_col_passes = json_number(text, "n_col_passes", &v) ? static_cast<uint32_t>(v) : 1;
    cfg.wgp_mode = text.find("\"wgp\":true") != std::string::npos;
    cfg.swap_grid = text.find("\"swap\":true") != std::string::npos;
    *c = cfg;
    if (tflops) *tflops = static_cast<float>(tf);
    return T0B_OK;
}

int32_t t0b_tune_cache_invalidate(const char* dir, uint32_t m, uint32_t n, uint32_t k) {
    std::remove(tune_path(dir, m, n, k).c_str());
    t0b::tuned_forget(m, n, k);   // and what this process measured for the shape (GemmTuner::invalidate, auto_gemm.rs:394-397)
    return T0B_OK;
}

int32_t t0b_set_autotune_dir(t0b_ctx* ctx, const char* dir) {
    if (!ctx) return T0B_ERR_INVALID;
    ctx->autotune_dir = (dir && !*dir) ? std::string() : tune_dir(dir);
    return T0B_OK;
}

const char* t0b_version(void) { return "t0b200 0.1 (sm_100a)"; }

}  // extern "C"
