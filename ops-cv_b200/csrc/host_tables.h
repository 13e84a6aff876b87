// Host-side evaluation of the per-axis tables that tables.cu builds on the device. The expressions are the same
// IEEE single-precision operations in the same order (this file is compiled with floating-point contraction off),
// so the integers and weights are bit-identical to the device tables; tests compare the two through
// opscvDebugAxisTable. The host copies are used only for planning: exact shared-memory tile sizes, tap bounds,
// and recognising regular patterns (integer up-scaling) that have dedicated kernels. Kernels always read the
// device tables.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <vector>

namespace opscv {
namespace host {

inline std::vector<int32_t> NearestSrc(int32_t in, int32_t out, float scale, bool exact = false)
{
    std::vector<int32_t> src(static_cast<size_t>(out));
    const long long last = in - 1;
    for (int32_t d = 0; d < out; ++d) {
        const float pos = exact ? static_cast<float>(d) + 0.5f : static_cast<float>(d);
        const long long s = static_cast<long long>(std::floor(pos * scale));
        src[d] = static_cast<int32_t>(s < last ? s : last);
    }
    return src;
}

struct Ranges {
    std::vector<int32_t> start, end;
};

inline Ranges NearestBwdRanges(int32_t in, int32_t out, float scale, bool exact = false)
{
    Ranges r;
    r.start.resize(in);
    r.end.resize(in);
    const float inv = 1.0f / scale;
    const long long lim = out;
    for (int32_t y = 0; y < in; ++y) {
        long long a, b;
        if (exact) {
            a = static_cast<long long>(std::ceil(static_cast<float>(y) * scale - 0.5f));
            b = static_cast<long long>(std::ceil(static_cast<float>(y + 1) * scale - 0.5f));
        } else {
            a = static_cast<long long>(std::ceil(static_cast<float>(y) * inv));
            b = static_cast<long long>(std::ceil(static_cast<float>(y + 1) * inv));
        }
        a = std::max<long long>(0, std::min(a, lim));
        b = std::max(a, std::min(b, lim));
        r.start[y] = static_cast<int32_t>(a);
        r.end[y] = static_cast<int32_t>(b);
    }
    return r;
}

struct Lerp {
    std::vector<int32_t> lo, hi;
    std::vector<float> delta;
};

// variant 0 = forward formula, 1 = backward (scatter) formula; see LerpTableKernel in tables.cu.
inline Lerp LerpTable(int32_t in, int32_t out, float scale, bool halfPixel, int variant)
{
    Lerp t;
    t.lo.resize(out);
    t.hi.resize(out);
    t.delta.resize(out);
    const long long last = in - 1;
    for (int32_t d = 0; d < out; ++d) {
        if (variant == 0) {
            float src = halfPixel ? (static_cast<float>(d) + 0.5f) * scale - 0.5f : static_cast<float>(d) * scale;
            if (src < 0.0f) {
                src = 0.0f;
            }
            long long lo = (src > 0.0f) ? static_cast<long long>(std::floor(src)) : 0;
            lo = std::min(lo, last);
            long long hi = (src > 0.0f) ? static_cast<long long>(std::ceil(src)) : 0;
            hi = std::min(hi, last);
            t.lo[d] = static_cast<int32_t>(lo);
            t.hi[d] = static_cast<int32_t>(hi);
            t.delta[d] = src - std::floor(src);
        } else {
            const float offset = halfPixel ? 0.5f : 0.0f;
            float src = (static_cast<float>(d) + offset) * scale - offset;
            src = (src < 0.0f) ? 0.0f : src;
            long long lo = std::min(static_cast<long long>(std::floor(src)), last);
            const float delta = std::fmin(std::fmax(src - static_cast<float>(lo), 0.0f), 1.0f);
            const long long hi = (lo < last) ? lo + 1 : lo;
            t.lo[d] = static_cast<int32_t>(lo);
            t.hi[d] = static_cast<int32_t>(hi);
            t.delta[d] = delta;
        }
    }
    return t;
}

// For every input index y: grads indices i with lo[i] <= y <= hi[i] (see LerpBwdRangeKernel).
inline Ranges LerpBwdRanges(const Lerp& t, int32_t in)
{
    Ranges r;
    r.start.resize(in);
    r.end.resize(in);
    const int32_t out = static_cast<int32_t>(t.lo.size());
    for (int32_t y = 0; y < in; ++y) {
        const int32_t first = static_cast<int32_t>(std::lower_bound(t.hi.begin(), t.hi.end(), y) - t.hi.begin());
        const int32_t end = static_cast<int32_t>(std::upper_bound(t.lo.begin() + std::min(first, out), t.lo.end(), y) -
                                                 t.lo.begin());
        r.start[y] = first;
        r.end[y] = std::max(end, first);
    }
    return r;
}

// Longest weight list of one axis of the trilinear backward: the most grad_output indices whose lower tap is y - 1
// or y, over all grad_input indices y (see TrilinearBwdTableKernel in upsample_trilinear3d.cu).
inline int32_t TrilinearBwdTaps(int32_t in, int32_t out, float scale, bool align)
{
    std::vector<int32_t> perLower(static_cast<size_t>(in) + 1, 0); // perLower[i] = indices whose lower tap is i
    const long long last = in - 1;
    for (int32_t d = 0; d < out; ++d) {
        const float real = align ? scale * static_cast<float>(d)
                                 : std::fmax(scale * (static_cast<float>(d) + 0.5f) - 0.5f, 0.0f);
        const long long i0 = std::min(static_cast<long long>(real), last);
        ++perLower[static_cast<size_t>(i0)];
    }
    int32_t worst = 1;
    for (int32_t y = 0; y < in; ++y) {
        worst = std::max(worst, perLower[y] + (y > 0 ? perLower[y - 1] : 0));
    }
    return worst;
}

// Largest number of rows `need(h0, h1)` over all tiles of `tileRows` output rows.
template <typename F>
inline int32_t MaxBand(int32_t outRows, int32_t tileRows, F need)
{
    int32_t worst = 0;
    for (int32_t h0 = 0; h0 < outRows; h0 += tileRows) {
        worst = std::max(worst, need(h0, std::min(outRows, h0 + tileRows)));
    }
    return worst;
}

// Largest tileRows (<= outRows) whose worst band fits `budgetRows`; 0 if not even one output row fits.
template <typename F>
inline int32_t PickTileRows(int32_t outRows, int32_t budgetRows, F need)
{
    if (MaxBand(outRows, outRows, need) <= budgetRows) {
        return outRows;
    }
    int32_t lo = 0, hi = outRows; // invariant: lo fits (or 0), hi does not
    while (hi - lo > 1) {
        const int32_t mid = lo + (hi - lo) / 2;
        if (MaxBand(outRows, mid, need) <= budgetRows) {
            lo = mid;
        } else {
            hi = mid;
        }
    }
    return lo;
}

} // namespace host
} // namespace opscv
