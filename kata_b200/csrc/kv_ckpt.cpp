// KV segments of the engine's prefix-cache checkpoint file, read and written through the KV-plane calls of the C ABI.
// File format of the reference (src/ckpt.cpp:16-34): a 4 KiB header "BNSCKPT1" version 2, then 4 KiB-aligned segments:
// tokens, GDN state, conv state, per attention layer the KV planes (n rows of each plane, planes back to back), the MTP
// head's K and V rows, the last hidden state, the logits. This library owns only the KV and MTP-KV segments: it writes a
// file with the reference's header and segment offsets (the other segments are left as holes for the engine to fill) and
// restores the KV segments of any file with a matching header, as PrefixCache::restore does (src/ckpt.cpp:84-107):
// magic, version, model fingerprint, numerics tag, layer count, row size, both prefix hashes, the stored tokens and the
// exact file size are all checked before a byte reaches the cache; a short or mismatching file is rejected.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include "../../include/kata_attn.h"

namespace {

constexpr uint32_t kVersion = 2, kVocab = 248320, kMtpRow = KATA_KV_DIM * 2;
constexpr uint64_t kAlign = 4096, kHidBytes = 5120 * 4;

#pragma pack(push, 1)
struct Header {   // field order and widths of the reference's Hdr (src/ckpt.cpp:18-22); naturally aligned, so packing changes nothing
    char magic[8]; uint32_t version, n; uint64_t modelFp; char tag[64];
    uint32_t hasMtp, nAttn, kvRow, pad0; uint64_t gdnBytes, convBytes, hash0, hash1; int32_t lastTok, pad1;
    uint64_t tokensOff, gdnOff, convOff, kvOff, mtpOff, hOff, logitsOff, total;
};
#pragma pack(pop)
static_assert(sizeof(Header) == 8 + 4 + 4 + 8 + 64 + 16 + 32 + 8 + 64, "header layout");

uint64_t up(uint64_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

void layout(uint32_t n, uint64_t gdn, uint64_t conv, uint32_t nAttn, uint32_t kvRow, bool mtp, uint64_t* o /* 8 */) {
    o[0] = kAlign; o[1] = up(o[0] + 4ull * n); o[2] = up(o[1] + gdn); o[3] = up(o[2] + conv);
    o[4] = up(o[3] + (uint64_t)nAttn * n * kvRow); o[5] = up(o[4] + (mtp ? 2ull * n * kMtpRow : 0)); o[6] = up(o[5] + (mtp ? kHidBytes : 0));
    o[7] = o[6] + (uint64_t)kVocab * 4;
}

// two FNV-1a style streams over the token bytes (src/ckpt.cpp:36-39)
void prefix_hash(const int32_t* t, size_t n, uint64_t& a, uint64_t& b) {
    a = 1469598103934665603ull; b = 0x9E3779B97F4A7C15ull;
    for (size_t i = 0; i < n; i++) { const uint8_t* p = reinterpret_cast<const uint8_t*>(&t[i]); for (int k = 0; k < 4; k++) { a = (a ^ p[k]) * 1099511628211ull; b = (b ^ p[k] ^ 0x5bd1e995ull) * 0x100000001b3ull; } }
}

bool rd(int fd, void* buf, size_t len, uint64_t off) { uint8_t* p = (uint8_t*)buf; while (len) { ssize_t r = pread(fd, p, std::min<size_t>(len, 1u << 28), (off_t)off); if (r <= 0) return false; p += r; off += (uint64_t)r; len -= (size_t)r; } return true; }
bool wr(int fd, const void* buf, size_t len, uint64_t off) { const uint8_t* p = (const uint8_t*)buf; while (len) { ssize_t r = pwrite(fd, p, std::min<size_t>(len, 1u << 28), (off_t)off); if (r <= 0) return false; p += r; off += (uint64_t)r; len -= (size_t)r; } return true; }

uint32_t kv_row_sum(kata_attn_ctx* c) { uint32_t s = 0; for (int p = 0; p < kata_attn_kv_planes(c); p++) s += (uint32_t)kata_attn_kv_plane_row_bytes(c, p); return s; }

}  // namespace

extern "C" {

// Segment offsets {tokens, gdn, conv, kv, mtp, h, logits, total} of a checkpoint of n tokens (layoutFor, src/ckpt.cpp:30-34).
void kata_ckpt_layout(uint32_t n, uint64_t gdn_bytes, uint64_t conv_bytes, uint32_t n_attn, uint32_t kv_row, int has_mtp, uint64_t* out8) { layout(n, gdn_bytes, conv_bytes, n_attn, kv_row, has_mtp != 0, out8); }
void kata_ckpt_prefix_hash(const int32_t* tokens, uint32_t n, uint64_t* out2) { prefix_hash(tokens, n, out2[0], out2[1]); }

// Header and size checks of PrefixCache::restore (src/ckpt.cpp:91-96) without touching a cache: returns KATA_OK and the
// stored token count when `path` is a complete checkpoint of a prefix of `tokens` for this model / tag / geometry.
int kata_ckpt_probe(const char* path, const int32_t* tokens, uint32_t n_tokens, uint64_t model_fp, const char* tag, uint32_t n_attn, uint32_t kv_row, uint64_t gdn_bytes, uint64_t conv_bytes, int want_mtp, uint32_t* n_out) {
    if (!path || !tokens || !tag || !n_out) return KATA_ERR_ARG;
    *n_out = 0;
    int fd = open(path, O_RDONLY); if (fd < 0) return KATA_ERR_ARG;
    struct stat st; Header h; bool ok = fstat(fd, &st) == 0 && rd(fd, &h, sizeof h, 0);
    ok = ok && memcmp(h.magic, "BNSCKPT1", 8) == 0 && h.version == kVersion && h.n > 0 && h.n <= n_tokens && h.modelFp == model_fp && strncmp(h.tag, tag, sizeof h.tag) == 0 &&
         h.nAttn == n_attn && h.kvRow == kv_row && h.gdnBytes == gdn_bytes && h.convBytes == conv_bytes && (!want_mtp || h.hasMtp);
    if (ok) { uint64_t a, b; prefix_hash(tokens, h.n, a, b); ok = h.hash0 == a && h.hash1 == b; }
    uint64_t o[8];
    if (ok) { layout(h.n, h.gdnBytes, h.convBytes, h.nAttn, h.kvRow, h.hasMtp != 0, o); ok = (uint64_t)st.st_size == o[7]; }   // a truncated file fails here
    if (ok) { std::vector<int32_t> toks(h.n); ok = rd(fd, toks.data(), 4ull * h.n, o[0]) && memcmp(toks.data(), tokens, 4ull * h.n) == 0; }
    close(fd);
    if (!ok) return KATA_ERR_RANGE;
    *n_out = h.n;
    return KATA_OK;
}

// Writes a checkpoint file holding the header, the tokens and the KV (and MTP-KV) segments of the first n positions of
// sequence `seq`; the GDN, conv, hidden-state and logits segments are holes of the right size. The file is written as
// path.tmp and left there: with its valid header, hashes and size the reference's restore (src/ckpt.cpp:91-101) would accept
// it and load all-zero recurrent state and logits, so it must not appear under its final name before the engine has filled
// its own segments. kata_ckpt_publish then renames it, as the reference's writer does (src/ckpt.cpp:132-138).
int kata_ckpt_write_kv(kata_attn_ctx* trunk, kata_attn_ctx* mtp, int32_t seq, const char* path, const int32_t* tokens, uint32_t n, uint64_t model_fp, uint32_t n_attn,
                       uint64_t gdn_bytes, uint64_t conv_bytes, int32_t last_tok) {
    if (!trunk || !path || !tokens || n == 0) return KATA_ERR_ARG;
    const uint32_t kvRow = kv_row_sum(trunk); uint64_t o[8]; layout(n, gdn_bytes, conv_bytes, n_attn, kvRow, mtp != nullptr, o);
    Header h{}; memcpy(h.magic, "BNSCKPT1", 8); h.version = kVersion; h.n = n; h.modelFp = model_fp; strncpy(h.tag, kata_attn_numerics_tag(trunk), sizeof h.tag - 1);
    h.hasMtp = mtp ? 1 : 0; h.nAttn = n_attn; h.kvRow = kvRow; h.gdnBytes = gdn_bytes; h.convBytes = conv_bytes; prefix_hash(tokens, n, h.hash0, h.hash1); h.lastTok = last_tok;
    h.tokensOff = o[0]; h.gdnOff = o[1]; h.convOff = o[2]; h.kvOff = o[3]; h.mtpOff = o[4]; h.hOff = o[5]; h.logitsOff = o[6]; h.total = o[7];
    const std::string tmp = std::string(path) + ".tmp";
    int fd = open(tmp.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644); if (fd < 0) return KATA_ERR_ARG;
    bool ok = ftruncate(fd, (off_t)o[7]) == 0 && wr(fd, &h, sizeof h, 0) && wr(fd, tokens, 4ull * n, o[0]);
    std::vector<uint8_t> buf;
    for (uint32_t a = 0; ok && a < n_attn; a++) { uint64_t pre = 0;
        for (int pl = 0; ok && pl < kata_attn_kv_planes(trunk); pl++) { const uint64_t rb = kata_attn_kv_plane_row_bytes(trunk, pl); buf.resize((size_t)n * rb);
            ok = kata_attn_kv_plane_read(trunk, (int32_t)a, seq, pl, 0, (int32_t)n, buf.data()) == KATA_OK && wr(fd, buf.data(), buf.size(), o[3] + (uint64_t)n * ((uint64_t)a * kvRow + pre)); pre += rb; } }
    for (int v = 0; ok && mtp && v < 2; v++) { buf.resize((size_t)n * kMtpRow); ok = kata_attn_kv_plane_read(mtp, 0, seq, v, 0, (int32_t)n, buf.data()) == KATA_OK && wr(fd, buf.data(), buf.size(), o[4] + (uint64_t)v * n * kMtpRow); }
    ok = ok && fsync(fd) == 0;
    close(fd);
    if (!ok) { unlink(tmp.c_str()); return KATA_ERR_CUDA; }
    return KATA_OK;
}

int kata_ckpt_publish(const char* path) {
    if (!path) return KATA_ERR_ARG;
    const std::string tmp = std::string(path) + ".tmp";
    return rename(tmp.c_str(), path) == 0 ? KATA_OK : KATA_ERR_ARG;
}

// Restores the KV (and MTP-KV) segments of a checkpoint into sequence `seq` after the checks of kata_ckpt_probe. On any
// failure nothing is left half-restored: the caches are reset, as the reference does (src/ckpt.cpp:102).
int kata_ckpt_read_kv(kata_attn_ctx* trunk, kata_attn_ctx* mtp, int32_t seq, const char* path, const int32_t* tokens, uint32_t n_tokens, uint64_t model_fp, uint32_t n_attn,
                      uint64_t gdn_bytes, uint64_t conv_bytes, uint32_t* n_out) {
    if (!trunk || !n_out) return KATA_ERR_ARG;
    const uint32_t kvRow = kv_row_sum(trunk); uint32_t n = 0;
    int rc = kata_ckpt_probe(path, tokens, n_tokens, model_fp, kata_attn_numerics_tag(trunk), n_attn, kvRow, gdn_bytes, conv_bytes, mtp != nullptr, &n);
    if (rc != KATA_OK) return rc;
    uint64_t o[8]; layout(n, gdn_bytes, conv_bytes, n_attn, kvRow, true, o);
    int fd = open(path, O_RDONLY); if (fd < 0) return KATA_ERR_ARG;
    Header h; bool ok = rd(fd, &h, sizeof h, 0); if (ok) layout(n, gdn_bytes, conv_bytes, n_attn, kvRow, h.hasMtp != 0, o);
    std::vector<uint8_t> buf;
    for (uint32_t a = 0; ok && a < n_attn; a++) { uint64_t pre = 0;
        for (int pl = 0; ok && pl < kata_attn_kv_planes(trunk); pl++) { const uint64_t rb = kata_attn_kv_plane_row_bytes(trunk, pl); buf.resize((size_t)n * rb);
            ok = rd(fd, buf.data(), buf.size(), o[3] + (uint64_t)n * ((uint64_t)a * kvRow + pre)) && kata_attn_kv_plane_write(trunk, (int32_t)a, seq, pl, 0, (int32_t)n, buf.data()) == KATA_OK; pre += rb; } }
    for (int v = 0; ok && mtp && v < 2; v++) { buf.resize((size_t)n * kMtpRow); ok = rd(fd, buf.data(), buf.size(), o[4] + (uint64_t)v * n * kMtpRow) && kata_attn_kv_plane_write(mtp, 0, seq, v, 0, (int32_t)n, buf.data()) == KATA_OK; }
    close(fd);
    if (!ok) { kata_attn_reset(trunk, nullptr); if (mtp) kata_attn_reset(mtp, nullptr); return KATA_ERR_CUDA; }
    *n_out = n;
    return KATA_OK;
}

}  // extern "C"
