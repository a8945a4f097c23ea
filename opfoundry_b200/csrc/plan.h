// Host-side work planner: the metadata stage of the pipeline.
//
// Same job as the reference's get_mla_metadata_kernel (opus_attn/dsa_v32/common/
// get_mla_metadata.hpp:17-158): cut the KV work of every query into contiguous pieces so that
// all processors finish together, give every piece of a split unit a partial slot, and emit
// the tables the merge kernel walks.  The unit of cost here is one pipeline step of
// kTileRows top-k slots plus a fixed per-piece overhead (query load + epilogue), mirroring the
// reference's "kv blocks + fixed_overhead" cost (get_mla_metadata.hpp:27-37).  A work list
// belongs to one CTA pair (the two CTAs of a pair each accumulate one 256-column half of the
// output), so there are num_sms / 2 lists instead of the reference's 256 compute units.
//
// The plan depends only on shapes (and the optional per-query valid-length hint), never on the
// index values, so it is computed on the host and uploaded once per shape.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>
#include "defs.h"

namespace dsa {

constexpr int kPieceOverheadTiles = 6;  // cost of loading Q and writing the result, in tile steps
constexpr int kMinPieceTiles = 4;       // never cut a piece shorter than this

struct HostPlan {
    WorkspaceHeader hdr;
    std::vector<int32_t> list_indptr;
    std::vector<dsa_v32_work_info> works;
    std::vector<int32_t> reduce_indptr;
    std::vector<int32_t> reduce_slots;
    std::vector<ReduceDst> reduce_dst;
};

inline int64_t align256(int64_t x) { return (x + 255) & ~int64_t(255); }

// One unit of work = one (query row, head block), or one sequence whose s_q query rows share an index
// list and fit one 128-row tile together (stacked along the heads).
struct PlanUnit {
    int32_t q_row, head_block, stacked_rows, len;
};
inline void enumerate_units(const dsa_v32_shape& sh, std::vector<PlanUnit>& units) {
    const int n_hb = (sh.H + kHeadsPerBlock - 1) / kHeadsPerBlock;
    const bool can_stack = sh.mtp_shared != nullptr && sh.s_q > 1 && sh.s_q * sh.H <= kHeadsPerBlock && sh.H % 8 == 0;
    auto row_len = [&](int q) { return sh.valid_len_hint ? std::max(0, std::min(sh.topk, sh.valid_len_hint[q])) : sh.topk; };
    units.clear();
    for (int seq = 0; seq < sh.total_q / sh.s_q; ++seq) {
        const int q0 = seq * sh.s_q;
        if (can_stack && sh.mtp_shared[seq]) {
            int len = 0;
            for (int t = 0; t < sh.s_q; ++t) len = std::max(len, row_len(q0 + t));
            units.push_back(PlanUnit{q0, 0, sh.s_q, len});
            continue;
        }
        for (int t = 0; t < sh.s_q; ++t)
            for (int hb = 0; hb < n_hb; ++hb) units.push_back(PlanUnit{q0 + t, hb, 1, row_len(q0 + t)});
    }
}

// Header and byte offsets of a plan whose tables are filled in.
inline void finish_plan(const dsa_v32_shape& sh, int L, int n_hb, int next_slot, HostPlan& P) {
    WorkspaceHeader& h = P.hdr;
    std::memset(&h, 0, sizeof(h));
    h.magic = kWorkspaceMagic;
    h.total_q = sh.total_q;
    h.H = sh.H;
    h.topk = sh.topk;
    h.s_q = sh.s_q;
    h.num_lists = L;
    h.num_works = int(P.works.size());
    h.num_partials = next_slot;
    h.num_reduce_rows = int(P.reduce_dst.size());
    h.num_head_blocks = n_hb;
    h.has_stacked = 0;
    for (const auto& w : P.works)
        if (w.stacked_rows > 1) h.has_stacked = 1;
    int64_t off = 256;
    h.off_list_indptr = off;
    off = align256(off + int64_t(L + 1) * 4);
    h.off_works = off;
    off = align256(off + int64_t(P.works.size()) * sizeof(dsa_v32_work_info));
    h.off_reduce_indptr = off;
    off = align256(off + int64_t(P.reduce_indptr.size()) * 4);
    h.off_reduce_slots = off;
    off = align256(off + int64_t(std::max<size_t>(P.reduce_slots.size(), 1)) * 4);
    h.off_reduce_dst = off;
    off = align256(off + int64_t(std::max<size_t>(P.reduce_dst.size(), 1)) * sizeof(ReduceDst));
    h.off_o_accum = off;
    off = align256(off + int64_t(next_slot) * kHeadsPerBlock * kDV * 4);
    h.off_lse_accum = off;
    off = align256(off + int64_t(next_slot) * kHeadsPerBlock * 4);
    h.total_bytes = off;
}

// Balanced plan: every list gets the same cost; units are cut where a list's share ends.
inline int build_plan_split(const dsa_v32_shape& sh, int num_sms, HostPlan& P) {
    if (sh.total_q <= 0 || sh.H <= 0 || sh.topk <= 0 || sh.s_q <= 0) return DSA_V32_ERR_SHAPE;
    if (sh.total_q % sh.s_q != 0) return DSA_V32_ERR_SHAPE;
    if (num_sms < 2) return DSA_V32_ERR_SHAPE;
    const int L = num_sms / 2;
    const int n_hb = (sh.H + kHeadsPerBlock - 1) / kHeadsPerBlock;
    std::vector<PlanUnit> units;
    enumerate_units(sh, units);
    const int64_t n_units = int64_t(units.size());

    auto unit_len = [&](int64_t u) -> int { return units[size_t(u)].len; };
    auto unit_tiles = [&](int64_t u) -> int { return std::max(1, (unit_len(u) + kTileRows - 1) / kTileRows); };

    // Cost of a piece = its tile steps + a fixed overhead.  Every list is given an equal share of
    // what is still to be handed out (recomputed list by list, so rounding and the overhead added by
    // cuts never pile up in the last list).
    int64_t tiles_left = 0;
    for (int64_t u = 0; u < n_units; ++u) tiles_left += unit_tiles(u);

    P.list_indptr.assign(L + 1, 0);
    P.works.clear();
    P.reduce_indptr.assign(1, 0);
    P.reduce_slots.clear();
    P.reduce_dst.clear();

    int64_t u = 0;
    int cur_tile = 0;       // tiles of unit u already handed out
    int pieces_of_unit = 0; // pieces of unit u emitted so far
    int next_slot = 0;
    std::vector<int> open_piece_ids;  // work indices of the pieces of the unit being split

    auto emit = [&](int tile_begin, int tile_end, bool last_piece) {
        const int q = units[size_t(u)].q_row, hb = units[size_t(u)].head_block;
        const int len = std::max(unit_len(u), 1);
        dsa_v32_work_info w;
        std::memset(&w, 0, sizeof(w));
        w.q_row = q;
        w.head_block = hb;
        w.stacked_rows = units[size_t(u)].stacked_rows;
        w.k_begin = tile_begin * kTileRows;
        w.k_end = last_piece ? std::min(std::max(len, w.k_begin + 1), sh.topk) : tile_end * kTileRows;
        w.partial_slot = -1;
        w.reduce_row = -1;
        open_piece_ids.push_back(int(P.works.size()));
        P.works.push_back(w);
        ++pieces_of_unit;
        if (last_piece) {
            if (pieces_of_unit > 1) {
                const int rr = int(P.reduce_dst.size());
                for (int id : open_piece_ids) {
                    P.works[id].partial_slot = next_slot;
                    P.works[id].reduce_row = rr;
                    P.reduce_slots.push_back(next_slot++);
                }
                P.reduce_indptr.push_back(int(P.reduce_slots.size()));
                P.reduce_dst.push_back(ReduceDst{q, units[size_t(u)].stacked_rows > 1 ? -units[size_t(u)].stacked_rows : hb});
            }
            open_piece_ids.clear();
            pieces_of_unit = 0;
            cur_tile = 0;
            ++u;
        } else {
            cur_tile = tile_end;
        }
    };

    // With little work only as many lists are used as can each get a minimum-length piece; the rest
    // stay empty (their CTA pairs exit at once).
    int L_used = int(std::max<int64_t>(1, std::min<int64_t>(L, tiles_left / kMinPieceTiles)));
    if (sh.flags & DSA_V32_PLAN_AUTO_SPLIT) {
        // the reference's effective_splits (get_mla_metadata.hpp:8-13) with its coefficient 1.2 (defs.h:62):
        // the cost it takes the root of is "blocks + overhead" summed over the units
        const double work = double(std::max<int64_t>(1, tiles_left + n_units * kPieceOverheadTiles)) * double(L);
        const long eff = std::lrint(1.2 * std::sqrt(work));
        L_used = int(std::max<long>(1, std::min<long>(eff, L_used)));
    }
    for (int list = 0; list < L; ++list) {
        if (list >= L_used) {
            P.list_indptr[list + 1] = int(P.works.size());
            continue;
        }
        const bool last_list = (list == L_used - 1);
        // pieces still to come: one per unit plus one more for every list boundary that cuts a unit
        const int lists_left = L_used - list;
        const double left =
            double(tiles_left) + double(n_units - u + std::min<int64_t>(lists_left - 1, tiles_left / kMinPieceTiles)) * kPieceOverheadTiles;
        const double budget = left / double(lists_left);
        double used = 0.0;
        while (u < n_units) {
            const int tiles = unit_tiles(u);
            const int rem_tiles = tiles - cur_tile;
            const int piece_cost = rem_tiles + kPieceOverheadTiles;
            if (last_list || used + piece_cost <= budget + 0.5) {
                emit(cur_tile, tiles, true);
                used += piece_cost;
                tiles_left -= rem_tiles;
                continue;
            }
            // the share ends inside this unit: cut it, keeping both sides at least kMinPieceTiles long
            const int room = int(budget - used + 0.5) - kPieceOverheadTiles;
            const int take = std::min(room, rem_tiles - kMinPieceTiles);
            if (take >= kMinPieceTiles) {
                emit(cur_tile, cur_tile + take, false);
                tiles_left -= take;
                break;
            }
            // too short to cut: take it whole when more than half of it belongs here, else leave it
            if (2.0 * (budget - used) >= double(piece_cost)) {
                emit(cur_tile, tiles, true);
                tiles_left -= rem_tiles;
            }
            break;
        }
        P.list_indptr[list + 1] = int(P.works.size());
    }

    finish_plan(sh, L, n_hb, next_slot, P);
    return DSA_V32_OK;
}

// Largest cost (tile steps + per-piece overhead) any list of the plan carries.
inline int64_t plan_makespan(const HostPlan& P) {
    int64_t worst = 0;
    for (size_t l = 0; l + 1 < P.list_indptr.size(); ++l) {
        int64_t c = 0;
        for (int w = P.list_indptr[l]; w < P.list_indptr[l + 1]; ++w)
            c += (P.works[w].k_end - P.works[w].k_begin + kTileRows - 1) / kTileRows + kPieceOverheadTiles;
        worst = std::max(worst, c);
    }
    return worst;
}

// Plan without any split: whole units, longest first, each to the list that is least loaded so far.
// No partial results, no merge; its lists are less even than those of the balanced plan.
inline int build_plan_whole(const dsa_v32_shape& sh, int num_sms, HostPlan& P) {
    if (sh.total_q <= 0 || sh.H <= 0 || sh.topk <= 0 || sh.s_q <= 0) return DSA_V32_ERR_SHAPE;
    if (sh.total_q % sh.s_q != 0) return DSA_V32_ERR_SHAPE;
    if (num_sms < 2) return DSA_V32_ERR_SHAPE;
    const int L = num_sms / 2;
    const int n_hb = (sh.H + kHeadsPerBlock - 1) / kHeadsPerBlock;
    std::vector<PlanUnit> units;
    enumerate_units(sh, units);
    const int64_t n_units = int64_t(units.size());
    auto unit_len = [&](int64_t u) -> int { return units[size_t(u)].len; };
    std::vector<int64_t> order(n_units);
    for (int64_t u = 0; u < n_units; ++u) order[u] = u;
    std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return unit_len(a) > unit_len(b); });
    // (load, list) min-heap
    std::vector<std::pair<int64_t, int>> heap;
    for (int l = 0; l < L; ++l) heap.emplace_back(0, l);
    auto cmp = [](const std::pair<int64_t, int>& a, const std::pair<int64_t, int>& b) { return a > b; };
    std::make_heap(heap.begin(), heap.end(), cmp);
    std::vector<std::vector<dsa_v32_work_info>> per_list(L);
    for (int64_t k = 0; k < n_units; ++k) {
        const int64_t u = order[k];
        const int len = std::max(unit_len(u), 1);
        std::pop_heap(heap.begin(), heap.end(), cmp);
        auto& top = heap.back();
        dsa_v32_work_info w;
        std::memset(&w, 0, sizeof(w));
        w.q_row = units[size_t(u)].q_row;
        w.head_block = units[size_t(u)].head_block;
        w.stacked_rows = units[size_t(u)].stacked_rows;
        w.k_begin = 0;
        w.k_end = std::min(len, sh.topk);
        w.partial_slot = -1;
        w.reduce_row = -1;
        per_list[top.second].push_back(w);
        top.first += (len + kTileRows - 1) / kTileRows + kPieceOverheadTiles;
        std::push_heap(heap.begin(), heap.end(), cmp);
    }
    P.list_indptr.assign(L + 1, 0);
    P.works.clear();
    P.reduce_indptr.assign(1, 0);
    P.reduce_slots.clear();
    P.reduce_dst.clear();
    for (int l = 0; l < L; ++l) {
        for (const auto& w : per_list[l]) P.works.push_back(w);
        P.list_indptr[l + 1] = int(P.works.size());
    }
    finish_plan(sh, L, n_hb, 0, P);
    return DSA_V32_OK;
}

// The plan a shape gets: the balanced one, unless the plan without splits is nearly as even.  A split
// costs what the makespan does not show: fp32 partial results written and read back (4x the bytes of
// the bf16 output) and the merge after the attention kernel, together worth about kMergeCostTiles steps.
constexpr int kMergeCostTiles = 6;
inline int build_plan(const dsa_v32_shape& sh, int num_sms, HostPlan& P) {
    int rc = build_plan_split(sh, num_sms, P);
    if (rc) return rc;
    if (P.reduce_dst.empty()) return DSA_V32_OK;
    HostPlan W;
    rc = build_plan_whole(sh, num_sms, W);
    if (rc) return rc;
    if (plan_makespan(W) <= plan_makespan(P) + kMergeCostTiles) P = W;
    return DSA_V32_OK;
}

// Serialises header + tables (everything before the partial buffers) into `blob`.
inline int64_t plan_meta_bytes(const HostPlan& P) { return P.hdr.off_o_accum; }

inline void serialize_plan(const HostPlan& P, uint8_t* blob) {
    std::memset(blob, 0, size_t(plan_meta_bytes(P)));
    std::memcpy(blob, &P.hdr, sizeof(P.hdr));
    std::memcpy(blob + P.hdr.off_list_indptr, P.list_indptr.data(), P.list_indptr.size() * 4);
    std::memcpy(blob + P.hdr.off_works, P.works.data(), P.works.size() * sizeof(dsa_v32_work_info));
    std::memcpy(blob + P.hdr.off_reduce_indptr, P.reduce_indptr.data(), P.reduce_indptr.size() * 4);
    if (!P.reduce_slots.empty())
        std::memcpy(blob + P.hdr.off_reduce_slots, P.reduce_slots.data(), P.reduce_slots.size() * 4);
    if (!P.reduce_dst.empty())
        std::memcpy(blob + P.hdr.off_reduce_dst, P.reduce_dst.data(), P.reduce_dst.size() * sizeof(ReduceDst));
}

}  // namespace dsa
