// Root files: the KV section of the reference's on-disk prefix cache (M/session.rs:92-129) and its key
// (M/session.rs:61-66). Host-only code: no CUDA here.
//
// Layout, little endian: "MECHTA-ROOT-1\n", u64 p, u64 n_ssm, u64 n_kv, p x u32 token ids, then vectors, each
// a u64 count of 32-bit words followed by the words: n_ssm DeltaNet states, n_ssm conv states, then per
// attention layer the K words and the V words of rows [0, p) (f32 values, or f16 pairs kept as raw u32 words,
// M/engine.rs:791-795). This library writes n_ssm = 0 and skips the states of files that have them.
#include <errno.h>
#include <stdio.h>
#include <string.h>

#include <string>

#include "../../include/mechta_kv.h"

namespace mkv {
void set_error(const char *fmt, ...);
}
using mkv::set_error;

static const char HEADER[] = "MECHTA-ROOT-1\n";

static size_t kv_words(mkv_fmt fmt, uint64_t p) { return fmt == MKV_F32 ? p * 512u : p * 512u / 2u; }

extern "C" {

uint64_t mkv_root_key(const uint32_t *tokens, size_t n) {
    uint64_t h = 0xcbf29ce484222325ull;
    for (size_t i = 0; i < n; i++)
        for (int b = 0; b < 4; b++) {
            h ^= (uint64_t)((tokens[i] >> (8 * b)) & 0xffu);
            h *= 0x100000001b3ull;
        }
    return h;
}

mkv_status mkv_root_write(const char *path, mkv_fmt fmt, int n_layers, uint32_t p, const uint32_t *tokens,
                          const void *payload, size_t payload_bytes) {
    if (!path || !payload || (p > 0 && !tokens) || n_layers < 1) {
        set_error("bad argument to mkv_root_write");
        return MKV_ERR_INVALID;
    }
    const size_t words = kv_words(fmt, p);
    if (payload_bytes != 2u * (size_t)n_layers * words * 4u) {
        set_error("payload is %zu bytes, %d layers of %u rows are %zu", payload_bytes, n_layers, p,
                  2u * (size_t)n_layers * words * 4u);
        return MKV_ERR_FORMAT;
    }
    // written under a temporary name, then renamed (M/session.rs:96,108)
    const std::string tmp = std::string(path) + ".tmp";
    FILE *f = fopen(tmp.c_str(), "wb");
    if (!f) {
        set_error("cannot create %s: %s", tmp.c_str(), strerror(errno));
        return MKV_ERR_IO;
    }
    bool ok = fwrite(HEADER, 1, sizeof HEADER - 1, f) == sizeof HEADER - 1;
    const uint64_t head[3] = {p, 0, (uint64_t)n_layers};
    ok = ok && fwrite(head, 8, 3, f) == 3;
    ok = ok && (p == 0 || fwrite(tokens, 4, p, f) == p);
    const char *src = static_cast<const char *>(payload);
    for (int i = 0; ok && i < 2 * n_layers; i++) {
        const uint64_t n = words;
        ok = fwrite(&n, 8, 1, f) == 1 && (words == 0 || fwrite(src, 4, words, f) == words);
        src += words * 4u;
    }
    ok = (fclose(f) == 0) && ok;
    if (!ok || rename(tmp.c_str(), path) != 0) {
        set_error("writing %s failed: %s", path, strerror(errno));
        remove(tmp.c_str());
        return MKV_ERR_IO;
    }
    return MKV_OK;
}

mkv_status mkv_root_read(const char *path, mkv_fmt fmt, int n_layers, uint32_t *p_out, uint32_t *tokens_out,
                         size_t tokens_cap, void *payload, size_t payload_cap, size_t *payload_bytes) {
    if (!path || !p_out) {
        set_error("bad argument to mkv_root_read");
        return MKV_ERR_INVALID;
    }
    FILE *f = fopen(path, "rb");
    if (!f) {
        set_error("cannot open %s: %s", path, strerror(errno));
        return MKV_ERR_IO;
    }
    mkv_status st = MKV_OK;
    char head[sizeof HEADER - 1];
    uint64_t h3[3];
    auto bad = [&](const char *why) {
        set_error("%s: %s", path, why);
        st = MKV_ERR_FORMAT;
    };
    if (fread(head, 1, sizeof head, f) != sizeof head || memcmp(head, HEADER, sizeof head) != 0) bad("not a MECHTA-ROOT-1 file");
    else if (fread(h3, 8, 3, f) != 3) bad("truncated header");
    else if (h3[0] > (uint64_t)MKV_CTX_MAX) bad("row count out of range");
    else if (h3[2] != (uint64_t)n_layers) bad("number of attention layers differs from the cache");
    if (st == MKV_OK) {
        const uint64_t p = h3[0], ns = h3[1];
        *p_out = (uint32_t)p;
        const size_t words = kv_words(fmt, p);
        const size_t need = 2u * (size_t)n_layers * words * 4u;
        if (payload_bytes) *payload_bytes = need;
        if (tokens_out && tokens_cap < p) {
            set_error("%s holds %llu tokens, room for %zu", path, (unsigned long long)p, tokens_cap);
            st = MKV_ERR_INVALID;
        } else if (payload && payload_cap < need) {
            set_error("%s holds %zu payload bytes, room for %zu", path, need, payload_cap);
            st = MKV_ERR_INVALID;
        } else {
            if (tokens_out) {
                if (p && fread(tokens_out, 4, p, f) != p) bad("truncated token list");
            } else if (fseek(f, (long)(4 * p), SEEK_CUR) != 0) bad("truncated token list");
            // DeltaNet and conv states of the reference's files: skipped
            for (uint64_t i = 0; st == MKV_OK && i < 2 * ns; i++) {
                uint64_t n;
                if (fread(&n, 8, 1, f) != 1 || fseek(f, (long)(4 * n), SEEK_CUR) != 0) bad("truncated state vector");
            }
            char *dst = static_cast<char *>(payload);
            for (int i = 0; st == MKV_OK && i < 2 * n_layers; i++) {
                uint64_t n;
                if (fread(&n, 8, 1, f) != 1) bad("truncated KV vector");
                else if (n < words) bad("KV vector shorter than p rows of this format");
                else if (payload) {
                    // the reference reads back only the first data_words(p * 512) words (M/engine.rs:808-812)
                    if (words && fread(dst, 4, words, f) != words) bad("truncated KV vector");
                    else if (n > words && fseek(f, (long)(4 * (n - words)), SEEK_CUR) != 0) bad("truncated KV vector");
                    dst += words * 4u;
                } else if (fseek(f, (long)(4 * n), SEEK_CUR) != 0) bad("truncated KV vector");
            }
        }
    }
    fclose(f);
    return st;
}

} // extern "C"
