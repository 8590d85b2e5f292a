#pragma once
// Layout arithmetic for the Ulysses 4D all-to-all. Host-only and free of CUDA, torch and any
// communication library, so the whole addressing contract can be replayed on a CPU.
//
// The exchange is described from both ends. `sends` is what this rank pushes, one Route per
// destination peer; `recvs` is the mirror image, what each peer pushes into this rank's window.
// A device kernel walks `sends`; a pull-style consumer or a CPU executor that unpacks a receive
// buffer walks `recvs`. Uneven per-rank shards are the general case; even shards are the same code
// with equal entries.
//
// Parity: plays the role of include/fast_ulysses/a2a_plan.hpp:19-65 and src/a2a_plan.cc:143-216 of
// the reference, but emits per-peer routes for an SM kernel instead of cudaMemcpy2D/3D parameters.
#include <cstdint>
#include <string>
#include <vector>

namespace fu {

enum Mode : int {
    kScatterHeads = 0,  // (b, s_local, n_global, d) -> (b, s_global, n_local, d)
    kGatherHeads  = 1,  // (b, s_global, n_local, d) -> (b, s_local, n_global, d)
};

// The group's geometry. `seq[p]` / `heads[p]` are rank p's shard sizes, identical on every rank.
struct Geometry {
    int64_t              b     = 0;
    int64_t              d     = 0;
    int                  rank  = 0;
    int                  world = 0;
    std::vector<int64_t> seq;
    std::vector<int64_t> heads;

    int64_t seq_total() const;
    int64_t head_total() const;
    void    validate() const;  // throws std::invalid_argument naming the field
};

// A 3-level strided block move: `batches` x `rows` x `row_bytes`, byte offsets relative to the
// source tensor's base and the destination window's base.
struct Route {
    int     peer       = 0;  // sends: destination rank; recvs: source rank
    int64_t src_off    = 0;
    int64_t dst_off    = 0;
    int64_t src_pitch  = 0;  // bytes between consecutive rows at the source
    int64_t dst_pitch  = 0;
    int64_t row_bytes  = 0;
    int64_t rows       = 0;
    int64_t batches    = 1;
    int64_t src_batch  = 0;  // bytes between batch elements at the source
    int64_t dst_batch  = 0;
    int64_t bytes() const { return row_bytes * rows * batches; }
};

struct Plan {
    std::vector<int64_t> in_shape;      // what this rank must hand in
    std::vector<int64_t> out_shape;     // what this rank receives, dense from the window base
    int64_t              window_numel = 0;  // elements every rank's window must hold: max over ranks
    int64_t              out_numel    = 0;
    std::vector<Route>   sends;
    std::vector<Route>   recvs;
    // The parts of this rank's output that PEERS write (everything but the own share), as at most
    // two regions with src_off == dst_off relative to the window and to a caller-owned output
    // alike. A copying call sends the own share straight to the output and copies out only these.
    std::vector<Route>   from_peers;
};

// `in_strides` (elements, for dims b, s, n; the last dim must be dense and the head stride must be
// d) lets a caller hand in a view without densifying it; empty means contiguous.
Plan make_plan(const Geometry& g, int mode, int64_t elem_size,
               const std::vector<int64_t>& in_strides = {});

// The other rank's view of the same exchange: used to derive `recvs` and by tests.
Geometry as_rank(const Geometry& g, int rank);

}  // namespace fu
