// Host-side slot allocator for the token-indexed KV pool: the observable behaviour of the reference's
// LongServeMemoryManager (lowest free slot ids first, first free run for contiguous requests, int32 reference
// counts; loongserve/common/longserve_mem_manager.py:32-89) without touching the device: the free set is a
// bitmap scanned with count-trailing-zeros, so an allocation is a few microseconds of host work and needs
// no device-wide nonzero() / .item() round trip.
#include <stdint.h>
#include <string.h>

#include <vector>

#include "../../include/esp_attention.h"

struct esp_pool {
    int64_t size;
    int64_t free_count;
    std::vector<int32_t> refs;
    std::vector<uint64_t> free_bits;     // bit set = slot free
    int64_t first_free_word;             // no free bit below this word
};

static inline void set_free(esp_pool* p, int64_t i) { p->free_bits[i >> 6] |= (1ull << (i & 63)); }
static inline void clr_free(esp_pool* p, int64_t i) { p->free_bits[i >> 6] &= ~(1ull << (i & 63)); }
static inline bool is_free(const esp_pool* p, int64_t i) { return (p->free_bits[i >> 6] >> (i & 63)) & 1ull; }

extern "C" int esp_pool_create(int64_t size, esp_pool** out) {
    if (size <= 0 || !out) return ESP_ERR_BAD_ARG;
    esp_pool* p = new esp_pool();
    p->size = size;
    p->refs.assign((size_t)size, 0);
    p->free_bits.assign((size_t)((size + 63) >> 6), 0);
    for (int64_t i = 0; i < size; ++i) set_free(p, i);
    p->free_count = size;
    p->first_free_word = 0;
    *out = p;
    return ESP_OK;
}

extern "C" int esp_pool_destroy(esp_pool* p) {
    if (!p) return ESP_ERR_BAD_ARG;
    delete p;
    return ESP_OK;
}

extern "C" int64_t esp_pool_can_use(const esp_pool* p) { return p ? p->free_count : -1; }

// Lowest `n` free slots, ascending; each gets reference count 1.  ESP_ERR_TOO_LARGE when fewer are free.
extern "C" int esp_pool_alloc(esp_pool* p, int64_t n, int64_t* out) {
    if (!p || n < 0 || (n > 0 && !out)) return ESP_ERR_BAD_ARG;
    if (n > p->free_count) return ESP_ERR_TOO_LARGE;
    int64_t got = 0;
    const int64_t words = (int64_t)p->free_bits.size();
    for (int64_t w = p->first_free_word; w < words && got < n; ++w) {
        uint64_t bits = p->free_bits[w];
        while (bits && got < n) {
            const int b = __builtin_ctzll(bits);
            bits &= bits - 1;
            const int64_t slot = (w << 6) + b;
            out[got++] = slot;
            p->refs[slot] = 1;
        }
        p->free_bits[w] = bits;          // the bits not taken stay free
        if (bits == 0 && w == p->first_free_word) p->first_free_word = w + 1;
    }
    p->free_count -= n;
    return ESP_OK;
}

// First run of `n` consecutive free slots.  *start = -1 when no such run exists (nothing is allocated then).
extern "C" int esp_pool_alloc_contiguous(esp_pool* p, int64_t n, int64_t* start) {
    if (!p || n <= 0 || !start) return ESP_ERR_BAD_ARG;
    *start = -1;
    if (n > p->free_count) return ESP_OK;
    int64_t run = 0, run_start = 0;
    for (int64_t i = p->first_free_word << 6; i < p->size; ++i) {
        if ((i & 63) == 0 && run == 0 && p->free_bits[i >> 6] == 0) { i += 63; continue; }   // skip full words quickly
        if (is_free(p, i)) {
            if (run == 0) run_start = i;
            if (++run == n) {
                for (int64_t j = run_start; j <= i; ++j) { clr_free(p, j); p->refs[j] = 1; }
                p->free_count -= n;
                *start = run_start;
                return ESP_OK;
            }
        } else {
            run = 0;
        }
    }
    return ESP_OK;
}

extern "C" int esp_pool_add_refs(esp_pool* p, const int64_t* ids, int64_t n) {
    if (!p || n < 0 || (n > 0 && !ids)) return ESP_ERR_BAD_ARG;
    for (int64_t i = 0; i < n; ++i)
        if (ids[i] < 0 || ids[i] >= p->size) return ESP_ERR_BAD_ARG;      // checked before anything changes
    for (int64_t i = 0; i < n; ++i) {
        const int64_t s = ids[i];
        if (p->refs[s]++ == 0) { clr_free(p, s); --p->free_count; }
    }
    return ESP_OK;
}

extern "C" int esp_pool_decrease_refs(esp_pool* p, const int64_t* ids, int64_t n) {
    if (!p || n < 0 || (n > 0 && !ids)) return ESP_ERR_BAD_ARG;
    // nothing is changed unless the whole request is valid; a slot may appear several times in `ids`
    for (int64_t i = 0; i < n; ++i) {
        const int64_t s = ids[i];
        if (s < 0 || s >= p->size || p->refs[s] <= 0) return ESP_ERR_BAD_ARG;
    }
    for (int64_t i = 0; i < n; ++i) {
        const int64_t s = ids[i];
        if (p->refs[s] <= 0) {        // released more often in this call than it was held: undo and refuse
            for (int64_t k = 0; k < i; ++k) {
                const int64_t u = ids[k];
                if (p->refs[u]++ == 0) { clr_free(p, u); --p->free_count; }
            }
            return ESP_ERR_BAD_ARG;
        }
        if (--p->refs[s] == 0) {
            set_free(p, s);
            ++p->free_count;
            if ((s >> 6) < p->first_free_word) p->first_free_word = s >> 6;
        }
    }
    return ESP_OK;
}

extern "C" int esp_pool_free_all(esp_pool* p) {
    if (!p) return ESP_ERR_BAD_ARG;
    memset(p->refs.data(), 0, sizeof(int32_t) * (size_t)p->size);
    for (auto& w : p->free_bits) w = 0;
    for (int64_t i = 0; i < p->size; ++i) set_free(p, i);
    p->free_count = p->size;
    p->first_free_word = 0;
    return ESP_OK;
}

extern "C" int esp_pool_state(const esp_pool* p, int32_t* out) {
    if (!p || !out) return ESP_ERR_BAD_ARG;
    memcpy(out, p->refs.data(), sizeof(int32_t) * (size_t)p->size);
    return ESP_OK;
}
