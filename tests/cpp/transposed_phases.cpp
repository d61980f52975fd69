// Host check of the index arithmetic behind the per-phase form of transposed convolutions (csrc/model.hpp:
// transposed_lead, transposed_phase) against the reference's definition (convolution.hpp:443-469): the input is
// spread by the stride, padded, and convolved with stride 1.  For every output position the set of (filter tap,
// input index) pairs that meet a real input sample must be the one the phase formula gives.  Prints "ok" or the first
// mismatch.
#include "model.hpp"

#include <cstdio>
#include <set>
#include <utility>

int main() {
    using namespace fdk;
    long checked = 0;
    for (int pad : {(int)PAD_VALID, (int)PAD_SAME})
        for (int k = 1; k <= 7; ++k)
            for (int s = 1; s <= 4; ++s)
                for (int n = 1; n <= 9; ++n) {
                    // geometry of one dimension as the plan compiler derives it (plan.cpp: emit_conv, conv_geom)
                    const int extra = (pad == PAD_SAME && s > 1) ? s - 1 : 0;
                    const int spread = s == 1 ? n : (n - 1) * s + 1 + extra;
                    const int pad_lo = pad == PAD_SAME ? (k - 1) / 2 : k - 1;
                    const int out = pad == PAD_SAME ? spread : spread + k - 1;
                    const int off = extra - extra / 2;
                    const int lead = transposed_lead(k, s, pad);
                    for (int o = 0; o < out; ++o) {
                        std::set<std::pair<int, int>> want, got;
                        for (int kk = 0; kk < k; ++kk) {
                            const int d = o + kk - pad_lo;  // position in the spread tensor
                            if (d < 0 || d >= spread) continue;
                            const int y = d - off;
                            if (y < 0 || y % s != 0 || y / s >= n) continue;
                            want.insert({kk, y / s});
                        }
                        const int p = o % s, q = o / s;
                        const TransposedPhase t = transposed_phase(k, s, lead, p);
                        for (int j = 0; j < t.taps; ++j) {
                            const int i = q + j + t.shift;
                            if (i < 0 || i >= n) continue;  // outside the input: the tensor map fills zeros
                            got.insert({t.k0 + s * j, i});
                        }
                        if (want != got) {
                            std::printf("mismatch: pad %d k %d s %d n %d output %d\n", pad, k, s, n, o);
                            return 1;
                        }
                        ++checked;
                    }
                }
    std::printf("ok %ld\n", checked);
    return 0;
}
