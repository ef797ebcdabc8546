// Host-only part of librns_b200: error text, modulus validation and the
// constants derived from a modulus list.  No device code here.
#include "rns_common.cuh"

#include <climits>
#include <numeric>

namespace rns {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

static int64_t mod_inverse(int64_t a, int64_t m) {
    // Extended Euclid; a and m coprime, result in [0, m).
    int64_t old_r = ((a % m) + m) % m, r = m, old_s = 1, s = 0;
    while (r != 0) {
        const int64_t q = old_r / r;
        int64_t t = old_r - q * r; old_r = r; r = t;
        t = old_s - q * s; old_s = s; s = t;
    }
    return ((old_s % m) + m) % m;
}

static int centred(int64_t v, int m) {
    v = ((v % m) + m) % m;
    return (int)(v > m / 2 ? v - m : v);
}

static int validate(const int32_t* moduli, int channels) {
    if (moduli == nullptr) return fail(RNS_ERR_INVALID_ARGUMENT, "moduli is NULL");
    if (channels <= 0) return fail(RNS_ERR_BAD_MODULI, "moduli must not be empty");
    if (channels > kMaxCh)
        return fail(RNS_ERR_UNSUPPORTED, "at most %d residue channels are supported", kMaxCh);
    for (int i = 0; i < channels; ++i)
        if (moduli[i] < 2 || moduli[i] > 255)
            return fail(RNS_ERR_BAD_MODULI, "every modulus must be in [2, 255]");
    for (int i = 0; i < channels; ++i)
        for (int j = i + 1; j < channels; ++j)
            if (std::gcd(moduli[i], moduli[j]) != 1)
                return fail(RNS_ERR_BAD_MODULI, "moduli are not pairwise coprime: %d, %d",
                            moduli[i], moduli[j]);
    return RNS_OK;
}

int build_plan(const int32_t* moduli, int channels, Plan* out) {
    if (int rc = validate(moduli, channels)) return rc;
    Plan& p = *out;
    memset(&p, 0, sizeof(p));
    p.channels = channels;
    p.encode_single_fold = 1;
    unsigned __int128 prod = 1;
    p.product[0] = 1;
    for (int i = 0; i < channels; ++i) {
        const int m = moduli[i];
        p.mod[i] = m;
        const uint64_t recip = (1ull << 32) / (uint64_t)m;
        p.recip[i] = recip > (uint64_t)INT_MAX ? INT_MAX : (int32_t)recip;
        p.ubias[i] = (uint32_t)m * (uint32_t)((1u << 31) / (uint32_t)m);
        p.modf[i] = (float)m;
        p.rcpf[i] = 1.0f / (float)m;
        const int half = m / 2;
        p.enc_hi[i] = (uint32_t)(127 - half) * 0x01010101u;
        p.enc_lo[i] = (uint32_t)half * 0x01010101u;
        if (m < 86) p.encode_single_fold = 0;
        prod *= (unsigned)m;
        if (prod > (unsigned __int128)INT64_MAX)
            return fail(RNS_ERR_OVERFLOW, "product(moduli) must fit signed int64");
        p.product[i + 1] = (int64_t)prod;
    }
    p.encode_fast = 1;
    for (int i = 0; i < channels; ++i)
        if (p.mod[i] >= 128) p.encode_fast = 0;
    for (int i = 0; i < channels; ++i) p.enc_mfold[i] = p.mod[i] <= 191 ? (uint32_t)p.mod[i] : 0u;
    for (int i = 0; i < channels; ++i)
        p.enc_mk[i] = p.encode_fast ? (uint32_t)p.mod[i] << 25 : (uint32_t)p.mod[i];
    for (int i = 0; i < channels; ++i) {
        const int m = p.mod[i];
        const int64_t place_mod = (int64_t)(p.product[i] % m);
        const int64_t inv = i == 0 ? 1 : mod_inverse(place_mod, m);
        p.gscale[i] = (float)centred(inv, m);
        for (int j = 0; j < i; ++j)
            p.gneg[i][j] = (float)centred(-((p.product[j] % m) * inv), m);
        p.place64[i] = p.product[i];
        if (i < 4) p.place32[i] = (uint32_t)p.product[i];
    }
    return RNS_OK;
}

}  // namespace rns

extern "C" {

const char* rns_last_error(void) { return rns::g_error; }

int rns_version(void) { return 100; }

int rns_host_constants(const int32_t* moduli, int channels, int64_t* reciprocals,
                       int32_t* pairwise_inverses, int64_t* modulus_product) {
    rns::Plan plan;
    if (int rc = rns::build_plan(moduli, channels, &plan)) return rc;
    for (int i = 0; i < channels; ++i) {
        if (reciprocals) reciprocals[i] = (int64_t)((1ull << 32) / (uint64_t)moduli[i]);
        if (pairwise_inverses)
            for (int j = 0; j < channels; ++j)
                pairwise_inverses[j * channels + i] =
                    j < i ? (int32_t)rns::mod_inverse(moduli[j], moduli[i]) : 0;
    }
    if (modulus_product) *modulus_product = plan.product[channels];
    return RNS_OK;
}

int rns_minimal_prefix_channels(const int32_t* moduli, int channels, int64_t absolute_bound,
                                int min_channels) {
    rns::Plan plan;
    if (int rc = rns::build_plan(moduli, channels, &plan)) return -rc;
    if (absolute_bound < 0)
        return -rns::fail(RNS_ERR_INVALID_ARGUMENT, "absolute_bound must be non-negative");
    if (min_channels < 2 || min_channels > channels)
        return -rns::fail(RNS_ERR_INVALID_ARGUMENT,
                          "min_channels must be between 2 and len(moduli)");
    for (int c = min_channels; c <= channels; ++c)
        if ((unsigned __int128)2 * (unsigned __int128)absolute_bound <
            (unsigned __int128)plan.product[c])
            return c;
    return -rns::fail(RNS_ERR_OVERFLOW,
                      "full moduli set cannot represent bound %lld; capacity=%lld",
                      (long long)absolute_bound, (long long)((plan.product[channels] - 1) / 2));
}

/* Host evaluation of the device arithmetic (see the header). */
int rns_host_reconstruct(const int32_t* sums, int64_t count, const int32_t* moduli, int channels,
                         int active, int64_t* out) {
    rns::Plan plan;
    if (int rc = rns::build_plan(moduli, channels, &plan)) return rc;
    if (!sums || !out || count < 0 || active < 1 || active > channels)
        return rns::fail(RNS_ERR_INVALID_ARGUMENT, "host_reconstruct: bad argument");
    for (int64_t i = 0; i < count; ++i) {
        int acc[rns::kMaxCh] = {0};
        for (int c = 0; c < channels; ++c) acc[c] = sums[(int64_t)c * count + i];
        const long long wide = rns::reconstruct<rns::kMaxCh>(acc, plan, active);
        if (channels <= 4) {
            int four[4] = {acc[0], acc[1], acc[2], acc[3]};
            const int narrow = rns::reconstruct32<4>(four, plan, active);
            if ((long long)narrow != wide)
                return rns::fail(RNS_ERR_INVALID_ARGUMENT,
                                 "32- and 64-bit reconstructions disagree at %lld: %d vs %lld",
                                 (long long)i, narrow, wide);
        }
        // The two-phase epilogue first replaces each sum by its canonical residue (packed
        // into a byte), then reconstructs from those: same integer.
        {
            int res[rns::kMaxCh] = {0};
            bool in_range = true;
            for (int c = 0; c < channels; ++c) {
                if (acc[c] > INT32_MAX - plan.mod[c] || acc[c] < -(INT32_MAX - plan.mod[c])) in_range = false;
                const uint32_t r = rns::canonical_residue(acc[c], plan.mod[c], plan.recip[c], plan.ubias[c]);
                const long long expect = (((long long)acc[c] % plan.mod[c]) + plan.mod[c]) % plan.mod[c];
                if (in_range && (long long)r != expect)
                    return rns::fail(RNS_ERR_INVALID_ARGUMENT, "canonical residue of %d mod %d is %u, expected %lld",
                                     acc[c], plan.mod[c], r, expect);
                res[c] = (int)r;
                // the lighter form the epilogue uses when every modulus is below 128
                const uint32_t loose = rns::nonneg_residue(acc[c], plan.mod[c], plan.recip[c], plan.ubias[c]);
                if (in_range && (loose >= 2u * (uint32_t)plan.mod[c] || (long long)(loose % (uint32_t)plan.mod[c]) != expect))
                    return rns::fail(RNS_ERR_INVALID_ARGUMENT, "non-negative residue of %d mod %d is %u", acc[c],
                                     plan.mod[c], loose);
                if (plan.encode_fast) res[c] = (int)loose;
            }
            if (in_range && rns::reconstruct<rns::kMaxCh>(res, plan, active) != wide)
                return rns::fail(RNS_ERR_INVALID_ARGUMENT, "reconstruction from canonical residues disagrees at %lld",
                                 (long long)i);
        }
        out[i] = wide;
    }
    return RNS_OK;
}

int rns_host_encode_centered_i8(const int8_t* values, int64_t count, const int32_t* moduli,
                                int channels, int8_t* out) {
    rns::Plan plan;
    if (int rc = rns::build_plan(moduli, channels, &plan)) return rc;
    if (!plan.encode_single_fold)
        return rns::fail(RNS_ERR_UNSUPPORTED, "the packed encoder needs every modulus >= 86");
    if (!values || !out || count < 0 || count % 4 != 0)
        return rns::fail(RNS_ERR_INVALID_ARGUMENT, "host_encode: count must be a multiple of 4");
    for (int64_t i = 0; i < count; i += 4) {
        uint32_t x;
        memcpy(&x, values + i, 4);
        const uint32_t u = x ^ 0x80808080u, ul = u & 0x7f7f7f7fu;
        for (int c = 0; c < channels; ++c) {
            const uint32_t y = plan.encode_fast
                ? rns::encode_word<true>(u, ul, plan.enc_hi[c], plan.enc_lo[c], plan.enc_mk[c])
                : rns::encode_word<false>(u, ul, plan.enc_hi[c], plan.enc_lo[c], plan.enc_mk[c]);
            memcpy(out + (int64_t)c * count + i, &y, 4);
        }
    }
    return RNS_OK;
}

int rns_host_encode_reduced_i8(const int8_t* values, int64_t count, const int32_t* moduli,
                               int channels, int8_t* out) {
    rns::Plan plan;
    if (int rc = rns::build_plan(moduli, channels, &plan)) return rc;
    if (!values || !out || count < 0 || count % 4 != 0)
        return rns::fail(RNS_ERR_INVALID_ARGUMENT, "host_encode: count must be a multiple of 4");
    for (int64_t i = 0; i < count; i += 4) {
        uint32_t x;
        memcpy(&x, values + i, 4);
        const uint32_t u = x ^ 0x80808080u, d = rns::fold_pattern(x);
        for (int c = 0; c < channels; ++c) {
            const uint32_t y = rns::encode_word_reduced(u, d, plan.enc_mfold[c]);
            memcpy(out + (int64_t)c * count + i, &y, 4);
        }
    }
    return RNS_OK;
}

}  // extern "C"
