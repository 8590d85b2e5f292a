#include "a2a_plan.hpp"

#include <algorithm>
#include <stdexcept>

namespace fu {
namespace {

[[noreturn]] void reject(const std::string& why)
{
    throw std::invalid_argument("fast_ulysses_b200: " + why);
}

int64_t mul_or_reject(int64_t a, int64_t b, const char* what)
{
    int64_t out = 0;
    if (__builtin_mul_overflow(a, b, &out)) {
        reject(std::string(what) + " overflows int64 (" + std::to_string(a) + " * " + std::to_string(b) + ")");
    }
    return out;
}

int64_t sum_or_reject(const std::vector<int64_t>& v, const char* what)
{
    int64_t total = 0;
    for (int64_t x : v) {
        if (__builtin_add_overflow(total, x, &total)) {
            reject(std::string(what) + " overflows int64");
        }
    }
    return total;
}

std::vector<int64_t> starts_of(const std::vector<int64_t>& sizes)
{
    std::vector<int64_t> out(sizes.size(), 0);
    for (size_t i = 1; i < sizes.size(); ++i) {
        out[i] = out[i - 1] + sizes[i - 1];
    }
    return out;
}

// The route rank `from` uses to push its share to rank `to`. Source strides are those of a dense
// tensor unless `strides` (b, s, n in bytes) says otherwise.
struct Strides {
    int64_t batch, row;
};

bool route_between(const Geometry& g, int mode, int64_t d_bytes, int from, int to, const Strides* src_strides,
                   Route& r)
{
    const std::vector<int64_t> s0 = starts_of(g.seq);
    const std::vector<int64_t> h0 = starts_of(g.heads);
    const int64_t              S  = g.seq_total();
    const int64_t              N  = g.head_total();
    if (mode == kScatterHeads) {
        // `from` keeps every sequence row it owns but only the head columns `to` owns; they land in
        // `to`'s (b, S, heads[to], d) window at `from`'s sequence offset, rows back to back.
        r.row_bytes = g.heads[to] * d_bytes;
        r.rows      = g.seq[from];
        r.src_off   = h0[to] * d_bytes;
        r.src_pitch = src_strides ? src_strides->row : N * d_bytes;
        r.src_batch = src_strides ? src_strides->batch : g.seq[from] * N * d_bytes;
        r.dst_off   = s0[from] * r.row_bytes;
        r.dst_pitch = r.row_bytes;
        r.dst_batch = S * r.row_bytes;
    }
    else {
        // `from` holds every sequence row for its own heads; `to` gets the rows it owns, placed at
        // `from`'s head offset inside `to`'s (b, seq[to], N, d) window.
        r.row_bytes = g.heads[from] * d_bytes;
        r.rows      = g.seq[to];
        r.src_pitch = src_strides ? src_strides->row : r.row_bytes;
        r.src_batch = src_strides ? src_strides->batch : S * r.row_bytes;
        r.src_off   = s0[to] * r.src_pitch;
        r.dst_off   = h0[from] * d_bytes;
        r.dst_pitch = N * d_bytes;
        r.dst_batch = g.seq[to] * N * d_bytes;
    }
    r.batches = g.b;
    return r.row_bytes > 0 && r.rows > 0;
}

}  // namespace

int64_t Geometry::seq_total() const
{
    return sum_or_reject(seq, "seq_splits total");
}

int64_t Geometry::head_total() const
{
    return sum_or_reject(heads, "head_splits total");
}

void Geometry::validate() const
{
    if (world <= 0) {
        reject("world_size must be positive, got " + std::to_string(world));
    }
    if (rank < 0 || rank >= world) {
        reject("rank " + std::to_string(rank) + " is outside a group of " + std::to_string(world));
    }
    if (b <= 0 || d <= 0) {
        reject("b and d must be positive, got b=" + std::to_string(b) + ", d=" + std::to_string(d));
    }
    if (static_cast<int>(seq.size()) != world) {
        reject("seq_splits has " + std::to_string(seq.size()) + " entries, expected " + std::to_string(world));
    }
    if (static_cast<int>(heads.size()) != world) {
        reject("head_splits has " + std::to_string(heads.size()) + " entries, expected " + std::to_string(world));
    }
    for (int p = 0; p < world; ++p) {
        if (seq[p] < 0) {
            reject("seq_splits[" + std::to_string(p) + "] is negative");
        }
        if (heads[p] < 0) {
            reject("head_splits[" + std::to_string(p) + "] is negative");
        }
    }
}

Geometry as_rank(const Geometry& g, int rank)
{
    Geometry out = g;
    out.rank     = rank;
    return out;
}

Plan make_plan(const Geometry& g, int mode, int64_t elem_size, const std::vector<int64_t>& in_strides)
{
    g.validate();
    if (elem_size <= 0) {
        reject("elem_size must be positive, got " + std::to_string(elem_size));
    }
    if (mode != kScatterHeads && mode != kGatherHeads) {
        reject("mode must be 0 (scatter heads) or 1 (gather heads), got " + std::to_string(mode));
    }
    const int64_t S = g.seq_total();
    const int64_t N = g.head_total();
    // Every byte quantity below is a product of a subset of these factors, so one bound covers all
    // of them; an empty axis counts as 1 because it removes a route, not a factor.
    int64_t bound = 1;
    for (int64_t f : {g.b, S, N, g.d, elem_size}) {
        bound = mul_or_reject(bound, std::max<int64_t>(f, 1), "the exchange in bytes");
    }
    const int64_t d_bytes = g.d * elem_size;
    const int64_t s_me    = g.seq[g.rank];
    const int64_t n_me    = g.heads[g.rank];

    Plan plan;
    if (mode == kScatterHeads) {
        plan.in_shape  = {g.b, s_me, N, g.d};
        plan.out_shape = {g.b, S, n_me, g.d};
    }
    else {
        plan.in_shape  = {g.b, S, n_me, g.d};
        plan.out_shape = {g.b, s_me, N, g.d};
    }
    plan.out_numel = plan.out_shape[0] * plan.out_shape[1] * plan.out_shape[2] * plan.out_shape[3];
    // Peer offsets only line up while every rank's window is the same size, so the window holds the
    // LARGEST rank's output. Every rank can compute that without talking: the splits are global.
    for (int p = 0; p < g.world; ++p) {
        const int64_t rows  = (mode == kScatterHeads) ? S : g.seq[p];
        const int64_t heads = (mode == kScatterHeads) ? g.heads[p] : N;
        plan.window_numel   = std::max(plan.window_numel, g.b * rows * heads * g.d);
    }

    Strides        strides{};
    const Strides* sp = nullptr;
    if (!in_strides.empty()) {
        if (in_strides.size() != 3) {
            reject("in_strides must name the batch, sequence and head strides");
        }
        if (in_strides[2] != g.d) {
            reject("the head stride must equal d: the head and channel axes travel as one run of bytes");
        }
        strides.batch = mul_or_reject(in_strides[0], elem_size, "the input batch stride in bytes");
        strides.row   = mul_or_reject(in_strides[1], elem_size, "the input row stride in bytes");
        sp            = &strides;
    }
    for (int p = 0; p < g.world; ++p) {
        Route out;
        out.peer = p;
        if (route_between(g, mode, d_bytes, g.rank, p, sp, out)) {
            plan.sends.push_back(out);
        }
        Route in;
        in.peer = p;
        if (route_between(g, mode, d_bytes, p, g.rank, nullptr, in)) {
            plan.recvs.push_back(in);
        }
    }
    // Complement of the own share inside the output.
    const std::vector<int64_t> s0 = starts_of(g.seq);
    const std::vector<int64_t> h0 = starts_of(g.heads);
    auto region = [&](int64_t off, int64_t row_bytes, int64_t rows, int64_t pitch, int64_t batch) {
        if (row_bytes <= 0 || rows <= 0) {
            return;
        }
        Route r;
        r.peer      = g.rank;
        r.src_off   = r.dst_off = off;
        r.src_pitch = r.dst_pitch = pitch;
        r.row_bytes = row_bytes;
        r.rows      = rows;
        r.batches   = g.b;
        r.src_batch = r.dst_batch = batch;
        plan.from_peers.push_back(r);
    };
    if (mode == kScatterHeads) {
        const int64_t w = n_me * d_bytes;  // rows of the output are w bytes, back to back
        region(0, w, s0[g.rank], w, S * w);
        region((s0[g.rank] + s_me) * w, w, S - s0[g.rank] - s_me, w, S * w);
    }
    else {
        const int64_t pitch = N * d_bytes;
        region(0, h0[g.rank] * d_bytes, s_me, pitch, s_me * pitch);
        region((h0[g.rank] + n_me) * d_bytes, (N - h0[g.rank] - n_me) * d_bytes, s_me, pitch, s_me * pitch);
    }
    return plan;
}

}  // namespace fu
