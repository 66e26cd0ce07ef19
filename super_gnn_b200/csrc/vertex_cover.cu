// Minimum vertex cover of a bipartite graph (host code): Hopcroft-Karp maximum matching, then
// Koenig's construction from the unmatched LEFT vertices: with Z = everything reachable from them
// along alternating paths, the cover is (L \ Z) u (R n Z).  By the Dulmage-Mendelsohn
// decomposition this cover does not depend on which maximum matching was found.
//
// Set-up code of the pre/post-aggregation mode: for every (source rank, destination rank) pair the
// cross edges form a bipartite graph (left = source nodes, right = destination nodes); a source in
// the cover ships its raw row ("post"), any other edge is summed at the sender per destination
// ("pre"), so the rows on the wire number |cover|, the minimum possible.
#include <vector>

#include "common.cuh"

namespace sgnn {

struct HopcroftKarp {
    int64_t nL, nR;
    const int64_t *rowptr;
    const int32_t *col;
    std::vector<int32_t> matchL, matchR, dist;
    std::vector<int64_t> it;

    HopcroftKarp(int64_t nL_, int64_t nR_, const int64_t *rp, const int32_t *c)
        : nL(nL_), nR(nR_), rowptr(rp), col(c), matchL(nL_, -1), matchR(nR_, -1), dist(nL_, 0), it(nL_, 0) {}

    bool bfs()
    {
        std::vector<int32_t> queue;
        queue.reserve((size_t)nL);
        for (int64_t u = 0; u < nL; ++u) {
            if (matchL[u] < 0) {
                dist[u] = 0;
                queue.push_back((int32_t)u);
            } else {
                dist[u] = -1;
            }
        }
        bool found = false;
        for (size_t h = 0; h < queue.size(); ++h) {
            const int32_t u = queue[h];
            for (int64_t e = rowptr[u]; e < rowptr[u + 1]; ++e) {
                const int32_t w = matchR[col[e]];
                if (w < 0) {
                    found = true;
                } else if (dist[w] < 0) {
                    dist[w] = dist[u] + 1;
                    queue.push_back(w);
                }
            }
        }
        return found;
    }

    // iterative depth-first search for an augmenting path from the free left vertex `root`
    bool augment(int32_t root, std::vector<int32_t> &stack)
    {
        stack.clear();
        stack.push_back(root);
        while (!stack.empty()) {
            const int32_t u = stack.back();
            if (it[u] < rowptr[u + 1]) {
                const int32_t v = col[it[u]++];
                const int32_t w = matchR[v];
                if (w < 0) {
                    // free right vertex: flip the path held on the stack
                    int32_t vv = v;
                    for (int64_t i = (int64_t)stack.size() - 1; i >= 0; --i) {
                        const int32_t uu = stack[i];
                        const int32_t prev = matchL[uu];
                        matchL[uu] = vv;
                        matchR[vv] = uu;
                        vv = prev;
                    }
                    return true;
                }
                if (dist[w] == dist[u] + 1) stack.push_back(w);
            } else {
                dist[u] = -1;  // dead end in this phase
                stack.pop_back();
            }
        }
        return false;
    }

    int64_t run()
    {
        int64_t size = 0;
        // greedy start
        for (int64_t u = 0; u < nL; ++u) {
            for (int64_t e = rowptr[u]; e < rowptr[u + 1]; ++e) {
                if (matchR[col[e]] < 0) {
                    matchL[u] = col[e];
                    matchR[col[e]] = (int32_t)u;
                    ++size;
                    break;
                }
            }
        }
        std::vector<int32_t> stack;
        while (bfs()) {
            for (int64_t u = 0; u < nL; ++u) it[u] = rowptr[u];
            for (int64_t u = 0; u < nL; ++u)
                if (matchL[u] < 0 && augment((int32_t)u, stack)) ++size;
        }
        return size;
    }
};

}  // namespace sgnn

// Declared in include/supergnn_b200.h.  All pointers are HOST pointers.
extern "C" SGNN_API int sgnn_bipartite_min_vertex_cover(int64_t num_left, int64_t num_right, const int64_t *h_rowptr,
                                                        const int32_t *h_col, uint8_t *h_cover_left,
                                                        uint8_t *h_cover_right, int64_t *h_matching_size)
{
    using namespace sgnn;
    SGNN_REQUIRE(num_left >= 0 && num_right >= 0, SGNN_ERR_INVALID_ARGUMENT, "min_vertex_cover: negative size");
    SGNN_REQUIRE(num_left <= 2147483647LL && num_right <= 2147483647LL, SGNN_ERR_TOO_LARGE,
                 "min_vertex_cover: vertex counts must fit int32");
    SGNN_REQUIRE(h_rowptr && h_cover_left && h_cover_right, SGNN_ERR_INVALID_ARGUMENT, "min_vertex_cover: null pointer");
    SGNN_REQUIRE(h_rowptr[num_left] == 0 || h_col != nullptr, SGNN_ERR_INVALID_ARGUMENT, "min_vertex_cover: col is null");
    for (int64_t e = 0; e < h_rowptr[num_left]; ++e)
        SGNN_REQUIRE(h_col[e] >= 0 && h_col[e] < num_right, SGNN_ERR_INVALID_ARGUMENT,
                     "min_vertex_cover: column %d out of range at position %lld", h_col[e], (long long)e);
    HopcroftKarp hk(num_left, num_right, h_rowptr, h_col);
    const int64_t size = hk.run();
    if (h_matching_size) *h_matching_size = size;
    // Z: reachable from free left vertices by alternating paths (non-matching edge L->R, matching edge R->L)
    std::vector<uint8_t> seenL((size_t)num_left, 0), seenR((size_t)num_right, 0);
    std::vector<int32_t> queue;
    for (int64_t u = 0; u < num_left; ++u)
        if (hk.matchL[u] < 0) {
            seenL[u] = 1;
            queue.push_back((int32_t)u);
        }
    for (size_t h = 0; h < queue.size(); ++h) {
        const int32_t u = queue[h];
        for (int64_t e = h_rowptr[u]; e < h_rowptr[u + 1]; ++e) {
            const int32_t v = h_col[e];
            if (hk.matchL[u] == v || seenR[v]) continue;
            seenR[v] = 1;
            const int32_t w = hk.matchR[v];
            if (w >= 0 && !seenL[w]) {
                seenL[w] = 1;
                queue.push_back(w);
            }
        }
    }
    for (int64_t u = 0; u < num_left; ++u) h_cover_left[u] = seenL[u] ? 0 : 1;
    for (int64_t v = 0; v < num_right; ++v) h_cover_right[v] = seenR[v] ? 1 : 0;
    return SGNN_OK;
}
