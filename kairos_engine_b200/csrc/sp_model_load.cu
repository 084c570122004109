/* sp_model_load.cu — fills the resident arena straight from the reference's on-disk model format.
 *
 * Stands where the MoE share of build_weights (CF:2222-2372 of src/backends/cuda/cuda_forward.cu) and
 * moe_cache_init (CF:6773-6879) stood: walk the `.sp-model` tensor table, find each layer's router, norm
 * vectors, shared expert and packed expert tensors, and copy them into the arena (sp_moe_upload_layer).
 * File format (include/sp_engine/sp_model.h:97-134, little-endian, packed): a 512-byte header (magic "SPMD",
 * header_size 512, tensor_table_offset 512, tensor_data_offset a multiple of 65536, CRC-32 over its first 360
 * bytes) and 256-byte tensor entries sorted by xxh64(name). Dtypes used (sp_model.h:42-57): F32 = 1,
 * FROBENIUS_SCALE_FP32 = 12, OK_Q4B = 13 (nibble-packed codes), BLOCK_SCALE_FP16 = 14 (the "<weight>.bscale"
 * sibling). Checked: magic, layout rules, header CRC, every tensor's bounds, alignment, dtype, byte size against
 * the handle's geometry, and the name hash. NOT checked: the per-tensor blake3 digest (sp_model.h:131) - no
 * BLAKE3 implementation is part of this library.
 *
 * Tensor names: the reference's own loader is not in its tree, so the names are a table the caller may replace;
 * the defaults are GGUF-style "blk.<L>.<field>" names (CF:12191, 15091-15185) with the "<weight>.bscale" sibling
 * rule (sp_model.h:50-53).
 */
#include "../../include/sp_engine/moe_backend.h"
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

const sp_moe_config *sp_moe_config_of(const sp_moe *h);      /* api.cu */

namespace {

#pragma pack(push, 1)
struct Header {
    uint32_t magic; uint16_t vmaj, vmin; uint32_t header_size, arch_id, arch_used, arch_cap; uint8_t arch[256]; uint8_t tok_hash[32];
    uint32_t vocab, tensor_count; uint64_t table_off, data_off, file_size, created, transcoded; uint32_t crc; uint8_t reserved[148];
};
struct Entry {
    char name[80]; uint32_t dtype, n_dims; uint64_t dims[8]; uint64_t offset, size; uint32_t block_size, block_count; uint8_t blake3[32];
    uint64_t name_hash; uint8_t reserved[40];
};
#pragma pack(pop)
static_assert(sizeof(Header) == 512 && sizeof(Entry) == 256, "on-disk structs");

uint32_t crc32(const uint8_t *p, size_t n) {
    uint32_t c = 0xFFFFFFFFu;
    for (size_t i = 0; i < n; i++) { c ^= p[i]; for (int k = 0; k < 8; k++) c = (c >> 1) ^ (0xEDB88320u & (0u - (c & 1u))); }
    return ~c;
}
uint64_t rotl(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }
uint64_t rd64(const uint8_t *p) { uint64_t v; memcpy(&v, p, 8); return v; }
uint32_t rd32(const uint8_t *p) { uint32_t v; memcpy(&v, p, 4); return v; }
/* XXH64 (the table's sort key is xxh64(name, seed 0)) */
uint64_t xxh64(const uint8_t *p, size_t n) {
    const uint64_t P1 = 11400714785074694791ull, P2 = 14029467366897019727ull, P3 = 1609587929392839161ull, P4 = 9650029242287828579ull, P5 = 2870177450012600261ull;
    auto round = [&](uint64_t acc, uint64_t v) { return rotl(acc + v * P2, 31) * P1; };
    size_t i = 0; uint64_t h;
    if (n >= 32) {
        uint64_t v[4] = {P1 + P2, P2, 0, 0 - P1};
        for (; i + 32 <= n; i += 32) for (int k = 0; k < 4; k++) v[k] = round(v[k], rd64(p + i + 8 * k));
        h = rotl(v[0], 1) + rotl(v[1], 7) + rotl(v[2], 12) + rotl(v[3], 18);
        for (int k = 0; k < 4; k++) h = (h ^ round(0, v[k])) * P1 + P4;
    } else h = P5;
    h += n;
    for (; i + 8 <= n; i += 8) h = rotl(h ^ round(0, rd64(p + i)), 27) * P1 + P4;
    if (i + 4 <= n) { h = rotl(h ^ (rd32(p + i) * P1), 23) * P2 + P3; i += 4; }
    for (; i < n; i++) h = rotl(h ^ (p[i] * P5), 11) * P1;
    h ^= h >> 33; h *= P2; h ^= h >> 29; h *= P3; h ^= h >> 32;
    return h;
}

int fail(int code, const char *fmt, const char *path, const char *a = "", unsigned long long b = 0, unsigned long long c = 0) {
    char msg[640];
    snprintf(msg, sizeof msg, fmt, path, a, b, c);
    sp_set_error(msg);
    return code;
}

enum { kFields = 18 };
/* in the order of sp_moe_layer_weights without router_bias; %d = layer */
const char *kDefaultNames[kFields] = {
    "blk.%d.ffn_gate_inp.weight", "blk.%d.ffn_gate_inp.scale", "blk.%d.ffn_norm.weight", "blk.%d.post_ffw_norm_1.weight",
    "blk.%d.pre_ffw_norm_2.weight", "blk.%d.post_ffw_norm_2.weight", "blk.%d.post_ffw_norm.weight", "blk.%d.ffn_down_exps.scale",
    "blk.%d.ffn_gate_up_exps.weight", "blk.%d.ffn_gate_up_exps.weight.bscale", "blk.%d.ffn_down_exps.weight", "blk.%d.ffn_down_exps.weight.bscale",
    "blk.%d.ffn_gate.weight", "blk.%d.ffn_gate.weight.bscale", "blk.%d.ffn_up.weight", "blk.%d.ffn_up.weight.bscale",
    "blk.%d.ffn_down.weight", "blk.%d.ffn_down.weight.bscale"};
const char *kBiasName = "blk.%d.ffn_gate_inp.bias";      /* optional */

struct Mapped {
    const uint8_t *p = nullptr; size_t n = 0; int fd = -1;
    ~Mapped() { if (p) munmap((void *)p, n); if (fd >= 0) close(fd); }
};

}  // namespace

extern "C" int sp_moe_load_sp_model(sp_moe *h, const char *path, const char *const *names) {
    if (!h || !path) { sp_set_error("sp_moe_load_sp_model: NULL argument"); return SP_MOE_EBADARG; }
    const sp_moe_config &c = *sp_moe_config_of(h);
    if (!names) names = kDefaultNames;
    Mapped m;
    m.fd = open(path, O_RDONLY);
    struct stat st;
    if (m.fd < 0 || fstat(m.fd, &st) != 0) return fail(SP_MOE_EBADARG, "sp_moe_load_sp_model: cannot open %s", path);
    m.n = (size_t)st.st_size;
    if (m.n < sizeof(Header)) return fail(SP_MOE_EBADARG, "sp_moe_load_sp_model: %s is shorter than the 512-byte header", path);
    void *mp = mmap(nullptr, m.n, PROT_READ, MAP_PRIVATE, m.fd, 0);
    if (mp == MAP_FAILED) return fail(SP_MOE_ENOMEM, "sp_moe_load_sp_model: cannot map %s", path);
    m.p = (const uint8_t *)mp;
    Header hd; memcpy(&hd, m.p, sizeof hd);
    if (hd.magic != 0x444D5053u) return fail(SP_MOE_EBADARG, "sp_moe_load_sp_model: %s: bad magic (want 'SPMD')", path);
    if (hd.header_size != 512 || hd.table_off != 512 || hd.data_off % 65536 != 0)
        return fail(SP_MOE_EBADARG, "sp_moe_load_sp_model: %s: header size / table offset / data offset break the layout rules", path);
    if (crc32(m.p, 360) != hd.crc) return fail(SP_MOE_EBADARG, "sp_moe_load_sp_model: %s: header CRC mismatch", path);
    if (hd.file_size != m.n || hd.table_off + (uint64_t)hd.tensor_count * sizeof(Entry) > hd.data_off || hd.data_off > m.n)
        return fail(SP_MOE_EBADARG, "sp_moe_load_sp_model: %s: file size / tensor table do not fit the file", path);
    const Entry *tab = reinterpret_cast<const Entry *>(m.p + hd.table_off);      /* 512-byte offset: aligned for the packed struct */

    auto find = [&](const char *name, uint32_t dt_a, uint32_t dt_b, size_t want_bytes, const void **out, bool optional) -> int {
        const uint64_t key = xxh64((const uint8_t *)name, strlen(name));
        size_t lo = 0, hi = hd.tensor_count;                 /* the table is sorted by the name hash */
        while (lo < hi) { const size_t mid = (lo + hi) / 2; if (tab[mid].name_hash < key) lo = mid + 1; else hi = mid; }
        const Entry *e = nullptr;
        for (size_t i = lo; i < hd.tensor_count && tab[i].name_hash == key; i++)
            if (strncmp(tab[i].name, name, sizeof tab[i].name) == 0) { e = &tab[i]; break; }
        if (!e) { *out = nullptr; return optional ? SP_MOE_OK : fail(SP_MOE_EBADARG, "sp_moe_load_sp_model: %s: tensor '%s' is not in the table", path, name); }
        if (e->dtype != dt_a && e->dtype != dt_b) return fail(SP_MOE_EBADARG, "sp_moe_load_sp_model: %s: tensor '%s' has dtype %llu, not what the MoE path stores there", path, name, e->dtype);
        if (e->offset % 64 != 0 || hd.data_off + e->offset + e->size > m.n) return fail(SP_MOE_EBADARG, "sp_moe_load_sp_model: %s: tensor '%s' is misaligned or lies outside the file", path, name);
        if (e->size != want_bytes) return fail(SP_MOE_EBADARG, "sp_moe_load_sp_model: %s: tensor '%s' holds %llu bytes, the geometry needs %llu", path, name, e->size, want_bytes);
        *out = m.p + hd.data_off + e->offset;
        return SP_MOE_OK;
    };

    const size_t E = c.E, NE = c.NE, FFE = c.FFE, FFS = c.FFS;
    const size_t want[kFields] = {4 * NE * E, 4 * E, 4 * E, 4 * E, 4 * E, 4 * E, 4 * E, 4 * NE,
                                  NE * 2 * FFE * E / 2, 2 * NE * 2 * FFE * (E / 32), NE * E * FFE / 2, 2 * NE * E * (FFE / 32),
                                  FFS * E / 2, 2 * FFS * (E / 32), FFS * E / 2, 2 * FFS * (E / 32), E * FFS / 2, 2 * E * (FFS / 32)};
    const uint32_t dta[kFields] = {1, 1, 1, 1, 1, 1, 1, 12, 13, 14, 13, 14, 13, 14, 13, 14, 13, 14};
    const uint32_t dtb[kFields] = {1, 12, 1, 1, 1, 1, 1, 1, 13, 14, 13, 14, 13, 14, 13, 14, 13, 14};
    for (int L = 0; L < c.n_layers; L++) {
        const void *p[kFields]; char name[96];
        for (int f = 0; f < kFields; f++) {
            snprintf(name, sizeof name, names[f], L);
            const int rc = find(name, dta[f], dtb[f], want[f], &p[f], false);
            if (rc) return rc;
        }
        const void *bias = nullptr;
        snprintf(name, sizeof name, kBiasName, L);
        { const int rc = find(name, 1, 1, 4 * NE, &bias, true); if (rc) return rc; }
        sp_moe_layer_weights w;
        w.router_w = (const float *)p[0]; w.router_scale = (const float *)p[1]; w.router_bias = (const float *)bias;
        w.ffn_norm = (const float *)p[2]; w.post_ffw1 = (const float *)p[3]; w.pre_ffw2 = (const float *)p[4];
        w.post_ffw2 = (const float *)p[5]; w.post_ffw = (const float *)p[6]; w.dexps_scale = (const float *)p[7];
        w.gu_codes = (const uint8_t *)p[8]; w.gu_bs = (const uint16_t *)p[9]; w.dn_codes = (const uint8_t *)p[10]; w.dn_bs = (const uint16_t *)p[11];
        w.sg_codes = (const uint8_t *)p[12]; w.sg_bs = (const uint16_t *)p[13]; w.su_codes = (const uint8_t *)p[14]; w.su_bs = (const uint16_t *)p[15];
        w.sd_codes = (const uint8_t *)p[16]; w.sd_bs = (const uint16_t *)p[17];
        const int rc = sp_moe_upload_layer(h, L, &w);
        if (rc) return rc;
    }
    return SP_MOE_OK;
}
