// Host side of the tile_ir front end: TileGemm specs, their names, the size -> tile table, grids and kernarg blobs
// (src/t0/tile_ir.rs of the reference).  Nothing here touches the device; t0b_tile_dispatch lives with the GEMM launcher.
#include <algorithm>
#include <cstring>
#include <string>

#include "t0b_internal.hpp"

namespace {

t0b_tile_gemm make_tile(uint32_t tm, uint32_t tn, uint32_t tk, bool wgp = false, bool acc_swap = false) {
    t0b_tile_gemm s{};
    s.tile_m = tm;
    s.tile_n = tn;
    s.tile_k = tk;
    s.wgp_mode = wgp;
    s.double_buffer = 1;
    s.split_k = 1;
    s.swap_grid = 1;
    s.transpose = T0B_TILE_NT;
    s.acc_swap = acc_swap;
    s.n_epilogue = 0;
    return s;
}

struct NamedTile {
    const char* name;
    t0b_tile_gemm spec;
};

// TileGemm::tile_*(), src/t0/tile_ir.rs:119-316.  Only 128x128_k32 and the two 256x64 tiles run in WGP mode.
const NamedTile* tile_presets(size_t* count) {
    static const NamedTile list[] = {
        {"128x64_k16", make_tile(128, 64, 16)},
        {"64x64_k16", make_tile(64, 64, 16)},
        {"64x64_k32", make_tile(64, 64, 32)},
        {"64x64_k64", make_tile(64, 64, 64)},
        {"32x64_k16", make_tile(32, 64, 16)},
        {"128x64_k32", make_tile(128, 64, 32)},
        {"64x128_k32", make_tile(64, 128, 32)},
        {"64x128_k16", make_tile(64, 128, 16)},
        {"128x128_k16", make_tile(128, 128, 16)},
        {"128x128_k32", make_tile(128, 128, 32, true)},
        {"128x128_k48", make_tile(128, 128, 48)},
        {"128x128_k16_swap", make_tile(128, 128, 16, false, true)},
        {"128x128_k32_swap", make_tile(128, 128, 32, false, true)},
        {"256x64_k32_wgp", make_tile(256, 64, 32, true)},
        {"256x64_k64_wgp", make_tile(256, 64, 64, true)},
        {"128x128_k64", make_tile(128, 128, 64)},
        {"128x64_k64", make_tile(128, 64, 64)},
    };
    *count = sizeof(list) / sizeof(list[0]);
    return list;
}

t0b_tile_gemm preset_or_die(const char* name) {
    size_t n = 0;
    const NamedTile* list = tile_presets(&n);
    for (size_t i = 0; i < n; ++i)
        if (std::strcmp(list[i].name, name) == 0) return list[i].spec;
    return make_tile(64, 64, 16);
}

const char* epi_word(int32_t op) {
    switch (op) {
        case T0B_EPI_BIAS_ADD: return "bias";
        case T0B_EPI_SCALE: return "scale";
        case T0B_EPI_RELU: return "relu";
        case T0B_EPI_SILU: return "silu";
        case T0B_EPI_GELU_SIGMOID: return "gelu";
        case T0B_EPI_ABS: return "abs";
        case T0B_EPI_NEG: return "neg";
        case T0B_EPI_CLAMP: return "clamp";
        default: return nullptr;
    }
}

bool has_op(const t0b_tile_gemm* s, int32_t op) {
    for (uint32_t i = 0; i < s->n_epilogue && i < T0B_TILE_MAX_EPILOGUE; ++i)
        if (s->epilogue[i] == op) return true;
    return false;
}

void put_le(uint8_t* p, uint64_t v, int bytes) {
    for (int i = 0; i < bytes; ++i) p[i] = static_cast<uint8_t>(v >> (8 * i));
}

}  // namespace

namespace t0b {

bool tile_spec_valid(const t0b_tile_gemm* s) {
    if (!s || s->tile_m == 0 || s->tile_n == 0 || s->tile_k == 0) return false;
    if (s->tile_m % 32 != 0 || s->tile_n % 16 != 0 || s->tile_k % 16 != 0) return false;   // n_waves = tile_m / 32
    if (s->split_k == 0 || s->split_k > 16 || (s->split_k & (s->split_k - 1)) != 0) return false;
    if (s->transpose > T0B_TILE_NN || s->n_epilogue > T0B_TILE_MAX_EPILOGUE) return false;
    for (uint32_t i = 0; i < s->n_epilogue; ++i)
        if (!epi_word(s->epilogue[i])) return false;
    return true;
}

// Length of the kernarg blob a spec expects, and where its epilogue arguments sit.
size_t tile_kernarg_layout(const t0b_tile_gemm* s, size_t* bias_off, size_t* scale_off, size_t* clamp_off) {
    size_t off = 44;
    if (has_op(s, T0B_EPI_BIAS_ADD)) {
        off = (off + 7) & ~static_cast<size_t>(7);
        if (bias_off) *bias_off = off;
        off += 8;
    }
    if (has_op(s, T0B_EPI_SCALE)) {
        if (scale_off) *scale_off = off;
        off += 4;
    }
    if (has_op(s, T0B_EPI_CLAMP)) {
        if (clamp_off) *clamp_off = off;
        off += 8;
    }
    return off;
}

}  // namespace t0b

extern "C" {

int32_t t0b_tile_preset(const char* name, t0b_tile_gemm* out) {
    if (!name || !out) return T0B_ERR_INVALID;
    size_t n = 0;
    const NamedTile* list = tile_presets(&n);
    for (size_t i = 0; i < n; ++i)
        if (std::strcmp(list[i].name, name) == 0) {
            *out = list[i].spec;
            return T0B_OK;
        }
    return T0B_ERR_INVALID;
}

int32_t t0b_tile_name(const t0b_tile_gemm* s, char* buf, size_t cap) {
    if (!s || !buf || cap == 0) return T0B_ERR_INVALID;
    std::string name = "tile_gemm_" + std::to_string(s->tile_m) + "x" + std::to_string(s->tile_n) + "_k" + std::to_string(s->tile_k);
    if (s->double_buffer) name += "_db";
    if (s->split_k > 1) name += "_sk" + std::to_string(s->split_k);
    if (!s->swap_grid) name += "_mg";
    if (s->wgp_mode) name += "_wgp";
    if (s->transpose == T0B_TILE_NN) name += "_nn";
    if (s->acc_swap) name += "_swap";
    for (uint32_t i = 0; i < s->n_epilogue && i < T0B_TILE_MAX_EPILOGUE; ++i) {
        const char* w = epi_word(s->epilogue[i]);
        if (!w) return T0B_ERR_INVALID;
        name += "_";
        name += w;
    }
    if (name.size() + 1 > cap) return T0B_ERR_INVALID;
    std::memcpy(buf, name.c_str(), name.size() + 1);
    return static_cast<int32_t>(name.size());
}

uint32_t t0b_tile_wg_size(const t0b_tile_gemm* s) { return s ? (s->tile_m / 32) * 32 : 0; }

uint32_t t0b_tile_lds_total(const t0b_tile_gemm* s) {
    if (!s) return 0;
    const uint32_t per_buffer = s->tile_m * s->tile_k * 2 + s->tile_n * s->tile_k * 2;
    uint32_t total = s->double_buffer ? per_buffer * 2 : per_buffer;
    if (s->acc_swap) total += (s->tile_n / 16) * 8 * 32 * 4 * (s->tile_m / 32);   // one row block of accumulators per wave
    return total;
}

int32_t t0b_tile_auto_select(uint32_t m, uint32_t k, uint32_t n, uint32_t transpose, t0b_tile_gemm* out) {
    if (!out || transpose > T0B_TILE_NN) return T0B_ERR_INVALID;
    const uint32_t min_dim = std::min(m, n), max_dim = std::max(m, n);
    const bool k64 = k >= 64 && k % 64 == 0, k32 = k >= 32 && k % 32 == 0;
    t0b_tile_gemm s;
    if (min_dim >= 128 && max_dim >= 4096)
        s = preset_or_die(k64 ? "128x128_k64" : (k32 ? "128x128_k32" : "128x128_k16"));
    else if (min_dim >= 64 && max_dim >= 2048)
        s = preset_or_die((m >= 256 && k32) ? "256x64_k32_wgp" : (k32 ? "64x64_k32" : "64x64_k16"));
    else if (min_dim >= 64)
        s = preset_or_die(k64 ? "64x64_k64" : (k32 ? "64x64_k32" : "64x64_k16"));
    else if (m >= 32 || n >= 128)
        s = preset_or_die(k32 ? "64x64_k32" : "32x64_k16");
    else
        s = preset_or_die("32x64_k16");
    s.transpose = transpose;

    const uint32_t tiles = ((m + s.tile_m - 1) / s.tile_m) * ((n + s.tile_n - 1) / s.tile_n);
    const uint32_t k_iters = k / s.tile_k;
    uint32_t want;
    if (s.wgp_mode && tiles >= 96) want = 1;
    else if (tiles < 12) want = 8;
    else if (tiles < 48) want = 4;
    else if (k_iters > 16) want = std::max(1u, std::min(8u, k_iters / 8));
    else want = 1;
    if (want > 1 && k >= s.tile_k * 2) {
        uint32_t sk = std::min(want, k / s.tile_k);
        while (sk > 1 && k % (s.tile_k * sk) != 0) sk /= 2;
        if (sk > 1) s.split_k = sk;
    }
    *out = s;
    return T0B_OK;
}

int32_t t0b_tile_compute_grid(const t0b_tile_gemm* s, uint32_t m, uint32_t n, uint32_t grid[3]) {
    if (!t0b::tile_spec_valid(s) || !grid) return T0B_ERR_INVALID;
    const uint32_t wgs_n = (n + s->tile_n - 1) / s->tile_n, wgs_m = (m + s->tile_m - 1) / s->tile_m;
    const uint32_t wg = t0b_tile_wg_size(s);
    grid[0] = (s->swap_grid ? wgs_n : wgs_m) * wg;
    grid[1] = (s->swap_grid ? wgs_m : wgs_n) * s->split_k;
    grid[2] = 1;
    return T0B_OK;
}

int32_t t0b_tile_build_kernargs(const t0b_tile_gemm* s, uint64_t x, uint64_t wt, uint64_t y, uint32_t k, uint32_t n, uint32_t m,
                                uint64_t bias, float scale, float clamp_min, float clamp_max, uint8_t* out, size_t cap) {
    if (!t0b::tile_spec_valid(s) || !out) return T0B_ERR_INVALID;
    size_t bias_off = 0, scale_off = 0, clamp_off = 0;
    const size_t len = t0b::tile_kernarg_layout(s, &bias_off, &scale_off, &clamp_off);
    if (cap < len) return T0B_ERR_INVALID;
    std::memset(out, 0, len);
    uint32_t shift = 0;
    while ((1u << shift) < s->split_k) ++shift;
    put_le(out + 0, x, 8);
    put_le(out + 8, wt, 8);
    put_le(out + 16, y, 8);
    put_le(out + 24, k, 4);
    put_le(out + 28, n, 4);
    put_le(out + 32, shift, 4);
    put_le(out + 36, 0, 4);          // y_split_stride: always 0 on this path
    put_le(out + 40, m, 4);
    uint32_t bits;
    if (bias_off) put_le(out + bias_off, bias, 8);
    if (scale_off) {
        std::memcpy(&bits, &scale, 4);
        put_le(out + scale_off, bits, 4);
    }
    if (clamp_off) {
        std::memcpy(&bits, &clamp_min, 4);
        put_le(out + clamp_off, bits, 4);
        std::memcpy(&bits, &clamp_max, 4);
        put_le(out + clamp_off + 4, bits, 4);
    }
    return static_cast<int32_t>(len);
}

}  // extern "C"
