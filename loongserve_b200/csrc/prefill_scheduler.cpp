// Host-side search that groups newly arrived requests into prefill batches and gives each batch a run of
// instances, minimising the summed predicted iteration time weighted by the inverse request lengths — the search the
// reference runs before every prefill iteration (longserve_c_scheduler/src/main.cpp:12-87, called from
// router/manager.py:687-760).
//
// State: best[n][m] = least cost of serving the first n requests (sorted by length, longest first) on the first m
// instances (sorted by tokens in use); choice[n][m] = (size of the last batch, instances of the last batch).
// A batch of requests [n-b, n) on instances [m-u, m) is feasible when its tokens fit in the free tokens of those
// instances; its predicted time is A_u + B_u * sum(len) + C_u * sum(len^2) with one (A, B, C) row per ESP degree u.
// Two pruning rules of the reference are part of the observable result and are kept: the last batch is no larger
// than the one chosen for (n, m-1), and uses no fewer instances than the one chosen for (n-1, m); candidates are
// visited with b ascending and u descending, the search over u stops at the first infeasible u, and only a
// strictly smaller cost replaces the incumbent.
//
// esp_sched_minimize_prefill_iteration_time fills caller-owned tables exactly like the reference's function;
// esp_sched_plan_prefill does the whole job (prefix sums, search, choice of the instance count, back-tracking)
// in one call without any numpy temporaries.  Compile with floating-point contraction off: costs are compared
// bit for bit with the reference's.
#include <stdint.h>

#include <limits>
#include <vector>

#include "../../include/esp_attention.h"

namespace {

struct Prefix {
    const int64_t* p;
    // sum of elements [lo, hi) of the sequence whose inclusive prefix sums are p
    inline int64_t range(int64_t lo, int64_t hi) const { return p[hi - 1] - (lo > 0 ? p[lo - 1] : 0); }
};
struct PrefixF {
    const double* p;
    inline double range(int64_t lo, int64_t hi) const { return p[hi - 1] - (lo > 0 ? p[lo - 1] : 0.0); }
};

void search(int64_t R, int64_t I, double* best, int32_t* choice, Prefix tokens, Prefix squares, PrefixF inverse,
            Prefix room, const double* abc) {
    const int64_t W = I + 1;                                  // row length of both tables
    best[0] = 0.0;
    for (int64_t n = 1; n <= R; ++n) {
        for (int64_t m = 1; m <= I; ++m) {
            const int32_t cap_b = choice[(n * W + (m - 1)) * 2 + 0];
            const int64_t b_hi = cap_b != -1 ? cap_b : n;
            const int32_t floor_u = choice[((n - 1) * W + m) * 2 + 1];
            const int64_t u_lo = floor_u != -1 ? floor_u : 1;
            double* cell = best + n * W + m;
            int32_t* pick = choice + (n * W + m) * 2;
            for (int64_t b = 1; b <= b_hi; ++b) {
                const int64_t first_req = n - b;
                const int64_t need = tokens.range(first_req, n);
                const int64_t need_sq = squares.range(first_req, n);
                const double weight = inverse.range(first_req, n);
                for (int64_t u = m; u >= u_lo; --u) {
                    const int64_t first_inst = m - u;
                    if (need > room.range(first_inst, m)) break;              // fewer instances only have less room
                    const double* row = abc + u * 3;
                    const double batch_time = row[0] + row[1] * (double)need + row[2] * (double)need_sq;
                    const double total = batch_time * weight + best[first_req * W + first_inst];
                    if (total < *cell) {
                        *cell = total;
                        pick[0] = (int32_t)b;
                        pick[1] = (int32_t)u;
                    }
                }
            }
        }
    }
}

}  // namespace

extern "C" int esp_sched_minimize_prefill_iteration_time(int64_t num_new_req, int64_t num_instances, double* min_iteration_times,
                                                         int32_t* min_iteration_times_index, const int64_t* req_input_prefix_sum,
                                                         const int64_t* req_input_square_prefix_sum,
                                                         const double* inverted_req_input_prefix_sum,
                                                         const int64_t* left_token_prefix_sum, const double* predictor_parameters,
                                                         int64_t predictor_rows) {
    if (num_new_req < 0 || num_instances < 0 || !min_iteration_times || !min_iteration_times_index) return ESP_ERR_BAD_ARG;
    if (num_new_req > 0 && num_instances > 0 &&
        (!req_input_prefix_sum || !req_input_square_prefix_sum || !inverted_req_input_prefix_sum || !left_token_prefix_sum ||
         !predictor_parameters))
        return ESP_ERR_BAD_ARG;
    if (predictor_rows < num_instances + 1) return ESP_ERR_BAD_ARG;
    search(num_new_req, num_instances, min_iteration_times, min_iteration_times_index, Prefix{req_input_prefix_sum},
           Prefix{req_input_square_prefix_sum}, PrefixF{inverted_req_input_prefix_sum}, Prefix{left_token_prefix_sum},
           predictor_parameters);
    return ESP_OK;
}

extern "C" int esp_sched_plan_prefill(int64_t num_new_req, const int64_t* req_tokens, int64_t num_instances, const int64_t* left_tokens,
                                      const double* predictor_parameters, int64_t predictor_rows, int32_t* batch_sizes,
                                      int32_t* batch_instances, int64_t* num_batches, double* total_cost, double* max_iteration_time) {
    if (num_new_req <= 0 || num_instances <= 0 || !req_tokens || !left_tokens || !predictor_parameters || !batch_sizes ||
        !batch_instances || !num_batches)
        return ESP_ERR_BAD_ARG;
    if (predictor_rows < num_instances + 1) return ESP_ERR_BAD_ARG;
    const int64_t R = num_new_req, I = num_instances;
    std::vector<int64_t> tok(R), sq(R), room(I);
    std::vector<double> inv(R);
    int64_t t = 0, s = 0, r = 0;
    double v = 0.0;
    for (int64_t i = 0; i < R; ++i) {
        if (req_tokens[i] <= 0) return ESP_ERR_BAD_ARG;
        t += req_tokens[i];
        s += req_tokens[i] * req_tokens[i];
        v += 1.0 / (double)req_tokens[i];
        tok[i] = t; sq[i] = s; inv[i] = v;
    }
    for (int64_t i = 0; i < I; ++i) {
        if (left_tokens[i] < 0) return ESP_ERR_BAD_ARG;
        r += left_tokens[i];
        room[i] = r;
    }
    if (room[I - 1] < tok[R - 1]) return ESP_ERR_TOO_LARGE;           // the requests do not fit at all
    std::vector<double> best((size_t)((R + 1) * (I + 1)), std::numeric_limits<double>::infinity());
    std::vector<int32_t> choice((size_t)((R + 1) * (I + 1) * 2), -1);
    search(R, I, best.data(), choice.data(), Prefix{tok.data()}, Prefix{sq.data()}, PrefixF{inv.data()}, Prefix{room.data()},
           predictor_parameters);
    // fewest-cost instance count (first strict minimum), then walk the choices back from (R, m)
    const int64_t W = I + 1;
    double lowest = std::numeric_limits<double>::infinity();
    int64_t m = -1;
    for (int64_t k = 1; k <= I; ++k)
        if (best[R * W + k] < lowest) { lowest = best[R * W + k]; m = k; }
    if (m < 0) return ESP_ERR_UNSUPPORTED;                             // pruning left no feasible plan
    int64_t n = R, nb = 0;
    double longest = 0.0;
    while (n > 0) {
        const int32_t b = choice[(n * W + m) * 2 + 0], u = choice[(n * W + m) * 2 + 1];
        if (b == -1 || u == -1) return ESP_ERR_UNSUPPORTED;
        const Prefix T{tok.data()}, S{sq.data()};
        const double* row = predictor_parameters + (int64_t)u * 3;
        const double it = row[0] + row[1] * (double)T.range(n - b, n) + row[2] * (double)S.range(n - b, n);
        if (it > longest) longest = it;
        batch_sizes[nb] = b;
        batch_instances[nb] = u;
        ++nb;
        n -= b;
        m -= u;
    }
    if (m != 0) return ESP_ERR_UNSUPPORTED;
    *num_batches = nb;
    if (total_cost) *total_cost = lowest;
    if (max_iteration_time) *max_iteration_time = longest;
    return ESP_OK;
}
