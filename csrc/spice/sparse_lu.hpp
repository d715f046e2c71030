// Sparse LU that is analysed once and refactored many times.
//
// A transient run solves thousands of systems with one sparsity pattern and slowly changing values
// (every Newton iteration of every step). The work is therefore split the way circuit solvers split it:
//
//   analyse  (once per pattern, again only when a pivot degrades)
//            column order by minimum degree on the pattern of A + A^T, rows of very high degree (supply
//            nets) set aside and ordered last; row order by one elimination with threshold partial
//            pivoting on the current values (the diagonal is taken whenever it is within a factor 10 of
//            the largest candidate, so the minimum-degree order keeps its meaning; strict partial
//            pivoting is the second try when that is not stable enough); symbolic elimination
//            of the permuted pattern, which fixes the positions of every fill-in
//   refactor (every solve with new values; identical values reuse the factors) scatter the row-equilibrated values into the fixed pattern and eliminate row by
//            row without searching, allocating or pivoting
//   solve    two triangular sweeps, then iterative refinement against the original matrix with the same
//            factors while the componentwise backward error is above 1e-10
//
// A refactorisation that meets a tiny pivot, or a solve whose backward error does not come down, triggers a
// new analysis with the values of that moment. The reference densifies the matrix and runs Gaussian
// elimination on it for every solve (nangila-spice/nangila-node/src/gpu_solver.rs:22-330).
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <queue>
#include <set>
#include <utility>
#include <vector>

namespace nspice {

// Elimination order of the symmetric pattern (row_ptr, col) by minimum degree on the quotient graph: an eliminated
// vertex becomes an element that stands for the clique of its neighbours, a vertex keeps a list of plain neighbours
// and a list of elements, elements whose boundary is covered by a newer one are absorbed, and degrees are the usual
// upper bound |plain neighbours| + |boundary of the new element| + sum over the other elements of |boundary outside the
// new one| (no clique is ever written out, so the cost stays near the size of the factor). Vertices whose degree exceeds
// `dense_limit` are left out of the graph and come last, highest degree at the very end. Vertices flagged in `removed`
// are not part of the graph and not part of the result.
inline std::vector<int> minimum_degree_order(int n, const std::vector<int>& row_ptr, const std::vector<int>& col,
                                             const std::vector<char>& removed = {}) {
    auto out = [&](int v) { return !removed.empty() && removed[size_t(v)] != 0; };
    std::vector<std::vector<int>> adj(static_cast<size_t>(n)), elems(static_cast<size_t>(n)), boundary(static_cast<size_t>(n));
    for (int r = 0; r < n; ++r) {
        if (out(r)) continue;
        for (int k = row_ptr[size_t(r)]; k < row_ptr[size_t(r) + 1]; ++k) {
            int c = col[size_t(k)];
            if (c != r && !out(c)) { adj[size_t(r)].push_back(c); adj[size_t(c)].push_back(r); }
        }
    }
    for (auto& a : adj) { std::sort(a.begin(), a.end()); a.erase(std::unique(a.begin(), a.end()), a.end()); }
    const size_t dense_limit = std::max<size_t>(16, size_t(10.0 * std::sqrt(double(std::max(n, 1)))));
    std::vector<char> gone(static_cast<size_t>(n), 0);   // eliminated, removed or set aside as dense
    for (int v = 0; v < n; ++v) gone[size_t(v)] = out(v) ? 1 : 0;
    std::vector<std::pair<size_t, int>> dense;
    for (int v = 0; v < n; ++v)
        if (!gone[size_t(v)] && adj[size_t(v)].size() > dense_limit) { dense.emplace_back(adj[size_t(v)].size(), v); gone[size_t(v)] = 1; }
    if (!dense.empty())
        for (int v = 0; v < n; ++v) {
            auto& a = adj[size_t(v)];
            a.erase(std::remove_if(a.begin(), a.end(), [&](int u) { return gone[size_t(u)] != 0; }), a.end());
        }
    std::vector<size_t> degree(static_cast<size_t>(n), 0);
    std::set<std::pair<size_t, int>> queue;
    for (int v = 0; v < n; ++v)
        if (!gone[size_t(v)]) { degree[size_t(v)] = adj[size_t(v)].size(); queue.emplace(degree[size_t(v)], v); }
    std::vector<int> order;
    order.reserve(size_t(n));
    std::vector<char> element_alive(static_cast<size_t>(n), 0);
    std::vector<int> in_lp(static_cast<size_t>(n), -1);          // in_lp[v] == p: v belongs to the boundary being built for pivot p
    std::vector<long> outside(static_cast<size_t>(n), -1);       // per element: |boundary outside the new one|, valid when stamp matches
    std::vector<int> outside_stamp(static_cast<size_t>(n), -1);
    std::vector<int> lp;
    while (!queue.empty()) {
        if (queue.begin()->first + 1 >= queue.size()) {
            // what is left is (bounded by) a clique: any order gives the same fill
            for (auto& dv : queue) order.push_back(dv.second);
            break;
        }
        const int p = queue.begin()->second;
        queue.erase(queue.begin());
        gone[size_t(p)] = 1;
        order.push_back(p);
        // boundary of the new element: plain neighbours of p and the boundaries of p's elements, which it absorbs
        lp.clear();
        in_lp[size_t(p)] = p;
        for (int v : adj[size_t(p)])
            if (!gone[size_t(v)] && in_lp[size_t(v)] != p) { in_lp[size_t(v)] = p; lp.push_back(v); }
        for (int e : elems[size_t(p)]) {
            if (!element_alive[size_t(e)]) continue;
            for (int v : boundary[size_t(e)])
                if (!gone[size_t(v)] && in_lp[size_t(v)] != p) { in_lp[size_t(v)] = p; lp.push_back(v); }
            element_alive[size_t(e)] = 0;
            std::vector<int>().swap(boundary[size_t(e)]);
        }
        std::vector<int>().swap(adj[size_t(p)]);
        std::vector<int>().swap(elems[size_t(p)]);
        // for every element next to the boundary: how much of it lies outside (counted down from its size)
        for (int i : lp)
            for (int e : elems[size_t(i)]) {
                if (!element_alive[size_t(e)]) continue;
                if (outside_stamp[size_t(e)] != p) { outside_stamp[size_t(e)] = p; outside[size_t(e)] = long(boundary[size_t(e)].size()); }
                --outside[size_t(e)];
            }
        const size_t remaining = queue.size();
        for (int i : lp) {
            queue.erase({degree[size_t(i)], i});
            auto& a = adj[size_t(i)];
            a.erase(std::remove_if(a.begin(), a.end(), [&](int v) { return gone[size_t(v)] != 0 || in_lp[size_t(v)] == p; }), a.end());
            auto& el = elems[size_t(i)];
            size_t sum_outside = 0, keep = 0;
            for (int e : el) {
                if (!element_alive[size_t(e)]) continue;
                if (outside[size_t(e)] <= 0) { element_alive[size_t(e)] = 0; std::vector<int>().swap(boundary[size_t(e)]); continue; }  // covered by the new element
                sum_outside += size_t(outside[size_t(e)]);
                el[keep++] = e;
            }
            el.resize(keep);
            el.push_back(p);
            const size_t bound = a.size() + (lp.size() - 1) + sum_outside;
            degree[size_t(i)] = std::min({bound, degree[size_t(i)] + lp.size() - 1, remaining > 0 ? remaining - 1 : size_t(0)});
            queue.emplace(degree[size_t(i)], i);
        }
        boundary[size_t(p)] = lp;
        element_alive[size_t(p)] = 1;
    }
    std::sort(dense.begin(), dense.end());
    for (auto& d : dense) order.push_back(d.second);
    return order;
}

// Pivots that cost nothing: a column with a single entry (that entry's row can be eliminated without touching any
// other row) and a row with a single entry (its column is eliminated without fill). Found repeatedly on what is left;
// in a circuit matrix this removes every net held by an ideal source together with the source's branch current, and
// with them the supply rows that touch thousands of devices. Returns the (row, column) pairs in elimination order.
inline std::vector<std::pair<int, int>> singleton_pivots(int n, const std::vector<int>& row_ptr, const std::vector<int>& col) {
    std::vector<int> cptr(size_t(n) + 1, 0), crow(col.size());
    for (int c : col) ++cptr[size_t(c) + 1];
    for (int c = 0; c < n; ++c) cptr[size_t(c) + 1] += cptr[size_t(c)];
    {
        std::vector<int> fill(cptr.begin(), cptr.end() - 1);
        for (int r = 0; r < n; ++r)
            for (int k = row_ptr[size_t(r)]; k < row_ptr[size_t(r) + 1]; ++k) crow[size_t(fill[size_t(col[size_t(k)])]++)] = r;
    }
    std::vector<int> rcount(static_cast<size_t>(n)), ccount(static_cast<size_t>(n));
    std::vector<char> rdead(static_cast<size_t>(n), 0), cdead(static_cast<size_t>(n), 0);
    std::vector<std::pair<int, int>> work, out;  // (index, 0 = row / 1 = column)
    for (int i = 0; i < n; ++i) {
        rcount[size_t(i)] = row_ptr[size_t(i) + 1] - row_ptr[size_t(i)];
        ccount[size_t(i)] = cptr[size_t(i) + 1] - cptr[size_t(i)];
        if (ccount[size_t(i)] == 1) work.emplace_back(i, 1);
    }
    for (int i = 0; i < n; ++i)
        if (rcount[size_t(i)] == 1) work.emplace_back(i, 0);
    for (size_t w = 0; w < work.size(); ++w) {
        int r = -1, c = -1;
        if (work[w].second == 1) {
            c = work[w].first;
            if (cdead[size_t(c)] || ccount[size_t(c)] != 1) continue;
            for (int k = cptr[size_t(c)]; k < cptr[size_t(c) + 1]; ++k)
                if (!rdead[size_t(crow[size_t(k)])]) { r = crow[size_t(k)]; break; }
        } else {
            r = work[w].first;
            if (rdead[size_t(r)] || rcount[size_t(r)] != 1) continue;
            for (int k = row_ptr[size_t(r)]; k < row_ptr[size_t(r) + 1]; ++k)
                if (!cdead[size_t(col[size_t(k)])]) { c = col[size_t(k)]; break; }
        }
        if (r < 0 || c < 0) continue;
        rdead[size_t(r)] = cdead[size_t(c)] = 1;
        out.emplace_back(r, c);
        for (int k = row_ptr[size_t(r)]; k < row_ptr[size_t(r) + 1]; ++k) {
            const int cc = col[size_t(k)];
            if (!cdead[size_t(cc)] && --ccount[size_t(cc)] == 1) work.emplace_back(cc, 1);
        }
        for (int k = cptr[size_t(c)]; k < cptr[size_t(c) + 1]; ++k) {
            const int rr = crow[size_t(k)];
            if (!rdead[size_t(rr)] && --rcount[size_t(rr)] == 1) work.emplace_back(rr, 0);
        }
    }
    return out;
}

struct FactoredLuStats { uint64_t orderings = 0, analyses = 0, refactors = 0, reuses = 0, repivots = 0, refinement_rounds = 0; size_t factor_nnz = 0, singletons = 0; };

class FactoredLU {
public:
    FactoredLuStats stats;

    // Solves A x = rhs for the matrix given by (n, row_ptr, col, val). Returns false for a singular system.
    bool solve(int n, const std::vector<int>& row_ptr, const std::vector<int>& col, const std::vector<double>& val,
               const std::vector<double>& rhs, std::vector<double>& x) {
        if (n == 0) { x.clear(); return true; }
        if (valid_ && n == n_ && row_ptr == a_ptr_ && col == a_col_) {
            // a linear circuit at a fixed step presents the same values every time: the factors still stand
            if (factored_ && val == last_val_) {
                ++stats.reuses;
                if (solve_refined(val, rhs, x)) return true;
            }
            if (refactor(val) && solve_refined(val, rhs, x)) return true;
            ++stats.repivots;  // the row order chosen for earlier values no longer suits these
        }
        // threshold pivoting first (keeps the minimum-degree order, least fill); strict partial pivoting if that
        // is not stable enough for this matrix
        for (double threshold : {0.1, 1.0}) {
            if (!analyse(n, row_ptr, col, val, threshold)) continue;
            if (refactor(val) && solve_refined(val, rhs, x)) return true;
        }
        valid_ = false;
        return false;
    }

private:
    int n_ = 0;
    bool valid_ = false, order_ready_ = false, factored_ = false;
    std::vector<double> last_val_;
    std::vector<int> a_ptr_, a_col_;
    std::vector<int> q_, qinv_, p_, pinv_;       // position -> original column / row, and back
    std::vector<int> lu_ptr_, lu_col_, diag_;    // pattern of L + U in permuted indices, columns ascending
    std::vector<double> lu_val_, scale_, y_, res_, dx_;
    std::vector<int> a_to_lu_, pos_, prefer_;    // prefer_[k]: the row the ordering had in mind for column position k, or -1

    // ---- analysis -----------------------------------------------------------------------------------
    bool analyse(int n, const std::vector<int>& row_ptr, const std::vector<int>& col, const std::vector<double>& val, double threshold) {
        ++stats.analyses;
        valid_ = false;
        // free pivots first, minimum degree on what is left; the order depends on the pattern only, so a new
        // analysis of the same pattern (new row choice for new values) reuses it
        if (!(n == n_ && order_ready_ && row_ptr == a_ptr_ && col == a_col_)) {
            const auto single = singleton_pivots(n, row_ptr, col);
            std::vector<char> removed(static_cast<size_t>(n), 0), row_taken(static_cast<size_t>(n), 0);
            q_.clear();
            prefer_.assign(size_t(n), -1);
            for (auto& rc : single) {
                prefer_[q_.size()] = rc.first;
                q_.push_back(rc.second);
                removed[size_t(rc.second)] = 1;
                row_taken[size_t(rc.first)] = 1;
            }
            for (int c : minimum_degree_order(n, row_ptr, col, removed)) {
                if (!row_taken[size_t(c)]) prefer_[q_.size()] = c;
                q_.push_back(c);
            }
            stats.singletons = single.size();
            ++stats.orderings;
            order_ready_ = true;
        }
        n_ = n;
        a_ptr_ = row_ptr;
        a_col_ = col;
        qinv_.assign(size_t(n), 0);
        for (int j = 0; j < n; ++j) qinv_[size_t(q_[size_t(j)])] = j;
        if (!choose_rows(val, threshold)) return false;
        pinv_.assign(size_t(n), 0);
        for (int i = 0; i < n; ++i) pinv_[size_t(p_[size_t(i)])] = i;
        symbolic();
        a_to_lu_.assign(col.size(), -1);
        for (int r = 0; r < n; ++r) {
            const int i = pinv_[size_t(r)];
            auto b = lu_col_.begin() + lu_ptr_[size_t(i)], e = lu_col_.begin() + lu_ptr_[size_t(i) + 1];
            for (int k = row_ptr[size_t(r)]; k < row_ptr[size_t(r) + 1]; ++k) {
                auto it = std::lower_bound(b, e, qinv_[size_t(col[size_t(k)])]);
                a_to_lu_[size_t(k)] = int(it - lu_col_.begin());
            }
        }
        lu_val_.assign(lu_col_.size(), 0.0);
        scale_.assign(size_t(n), 1.0);
        pos_.assign(size_t(n), -1);
        stats.factor_nnz = lu_col_.size();
        valid_ = true;
        return true;
    }

    // One elimination with threshold partial pivoting, columns in the order q_: fills p_.
    bool choose_rows(const std::vector<double>& val, const double thr) {
        const int n = n_;
        using Row = std::vector<std::pair<int, double>>;
        std::vector<Row> rows(static_cast<size_t>(n));
        std::vector<std::vector<int>> col_rows(static_cast<size_t>(n));
        for (int r = 0; r < n; ++r) {
            Row& row = rows[size_t(r)];
            double mx = 0.0;
            for (int k = a_ptr_[size_t(r)]; k < a_ptr_[size_t(r) + 1]; ++k) {
                row.emplace_back(qinv_[size_t(a_col_[size_t(k)])], val[size_t(k)]);
                mx = std::max(mx, std::fabs(val[size_t(k)]));
            }
            std::sort(row.begin(), row.end());
            if (mx > 0.0)
                for (auto& e : row) e.second /= mx;
            for (auto& e : row) col_rows[size_t(e.first)].push_back(r);
        }
        auto entry = [](const Row& row, int c) -> double {
            auto it = std::lower_bound(row.begin(), row.end(), c, [](const std::pair<int, double>& p, int cc) { return p.first < cc; });
            return (it != row.end() && it->first == c) ? it->second : 0.0;
        };
        p_.assign(size_t(n), -1);
        std::vector<char> used(static_cast<size_t>(n), 0);
        Row merged;
        for (int k = 0; k < n; ++k) {
            auto& cands = col_rows[size_t(k)];
            std::sort(cands.begin(), cands.end());
            cands.erase(std::unique(cands.begin(), cands.end()), cands.end());
            double best = 0.0;
            for (int r : cands)
                if (!used[size_t(r)]) best = std::max(best, std::fabs(entry(rows[size_t(r)], k)));
            if (!(best > 1e-300)) return false;
            const int want = prefer_[size_t(k)];
            int p = -1;
            size_t plen = 0;
            if (want >= 0 && !used[size_t(want)] && std::fabs(entry(rows[size_t(want)], k)) >= thr * best) p = want;
            else
                for (int r : cands) {
                    if (used[size_t(r)]) continue;
                    double a = std::fabs(entry(rows[size_t(r)], k));
                    if (a >= thr * best && (p < 0 || rows[size_t(r)].size() < plen)) { p = r; plen = rows[size_t(r)].size(); }
                }
            used[size_t(p)] = 1;
            p_[size_t(k)] = p;
            const Row& prow = rows[size_t(p)];
            const double pv = entry(prow, k);
            for (int r : cands) {
                if (used[size_t(r)]) continue;
                Row& row = rows[size_t(r)];
                const double a = entry(row, k);
                if (a == 0.0) continue;
                const double f = a / pv;
                merged.clear();
                size_t i = 0, j = 0;
                while (i < row.size() || j < prow.size()) {
                    if (j >= prow.size() || (i < row.size() && row[i].first < prow[j].first)) merged.push_back(row[i++]);
                    else if (i >= row.size() || prow[j].first < row[i].first) {
                        if (prow[j].first > k) { merged.emplace_back(prow[j].first, -f * prow[j].second); col_rows[size_t(prow[j].first)].push_back(r); }
                        ++j;
                    } else {
                        if (row[i].first != k) merged.emplace_back(row[i].first, row[i].second - f * prow[j].second);
                        ++i; ++j;
                    }
                }
                row.swap(merged);
            }
        }
        return true;
    }

    // Pattern of L + U of the permuted matrix, row by row: a row starts as its own entries and takes over the
    // upper part of every earlier row it has an entry under.
    void symbolic() {
        const int n = n_;
        lu_ptr_.assign(size_t(n) + 1, 0);
        lu_col_.clear();
        diag_.assign(size_t(n), -1);
        std::vector<int> mark(static_cast<size_t>(n), -1), cols;
        std::priority_queue<int, std::vector<int>, std::greater<int>> lower;
        std::vector<std::vector<int>> upper(static_cast<size_t>(n));  // columns right of the diagonal, ascending
        for (int i = 0; i < n; ++i) {
            const int r = p_[size_t(i)];
            cols.clear();
            auto add = [&](int c) {
                if (mark[size_t(c)] == i) return;
                mark[size_t(c)] = i;
                cols.push_back(c);
                if (c < i) lower.push(c);
            };
            add(i);  // the pivot position exists even where A has a structural zero there
            for (int k = a_ptr_[size_t(r)]; k < a_ptr_[size_t(r) + 1]; ++k) add(qinv_[size_t(a_col_[size_t(k)])]);
            while (!lower.empty()) {
                const int k = lower.top();
                lower.pop();
                for (int c : upper[size_t(k)]) add(c);
            }
            std::sort(cols.begin(), cols.end());
            for (int c : cols) {
                if (c == i) diag_[size_t(i)] = int(lu_col_.size());
                if (c > i) upper[size_t(i)].push_back(c);
                lu_col_.push_back(c);
            }
            lu_ptr_[size_t(i) + 1] = int(lu_col_.size());
        }
    }

    // ---- numeric ------------------------------------------------------------------------------------
    bool refactor(const std::vector<double>& val) {
        ++stats.refactors;
        factored_ = false;
        const int n = n_;
        std::fill(lu_val_.begin(), lu_val_.end(), 0.0);
        for (int r = 0; r < n; ++r) {
            double mx = 0.0;
            for (int k = a_ptr_[size_t(r)]; k < a_ptr_[size_t(r) + 1]; ++k) mx = std::max(mx, std::fabs(val[size_t(k)]));
            const double s = mx > 0.0 ? 1.0 / mx : 1.0;
            scale_[size_t(r)] = s;
            for (int k = a_ptr_[size_t(r)]; k < a_ptr_[size_t(r) + 1]; ++k) lu_val_[size_t(a_to_lu_[size_t(k)])] = val[size_t(k)] * s;
        }
        for (int i = 0; i < n; ++i) {
            const int b = lu_ptr_[size_t(i)], e = lu_ptr_[size_t(i) + 1], d = diag_[size_t(i)];
            for (int t = b; t < e; ++t) pos_[size_t(lu_col_[size_t(t)])] = t;
            for (int t = b; t < d; ++t) {
                const int k = lu_col_[size_t(t)];
                const double lik = lu_val_[size_t(t)] / lu_val_[size_t(diag_[size_t(k)])];
                lu_val_[size_t(t)] = lik;
                if (lik == 0.0) continue;
                for (int u = diag_[size_t(k)] + 1; u < lu_ptr_[size_t(k) + 1]; ++u) lu_val_[size_t(pos_[size_t(lu_col_[size_t(u)])])] -= lik * lu_val_[size_t(u)];
            }
            for (int t = b; t < e; ++t) pos_[size_t(lu_col_[size_t(t)])] = -1;
            const double pv = std::fabs(lu_val_[size_t(d)]);
            if (!(pv > 1e-300) || !std::isfinite(pv)) return false;
        }
        last_val_ = val;
        factored_ = true;
        return true;
    }

    // x := A^-1 b through the factors (b in original row order, x in original column order).
    void apply(const std::vector<double>& b, std::vector<double>& x) {
        const int n = n_;
        y_.resize(size_t(n));
        for (int i = 0; i < n; ++i) {
            const int r = p_[size_t(i)];
            double acc = b[size_t(r)] * scale_[size_t(r)];
            for (int t = lu_ptr_[size_t(i)]; t < diag_[size_t(i)]; ++t) acc -= lu_val_[size_t(t)] * y_[size_t(lu_col_[size_t(t)])];
            y_[size_t(i)] = acc;
        }
        for (int i = n - 1; i >= 0; --i) {
            double acc = y_[size_t(i)];
            for (int t = diag_[size_t(i)] + 1; t < lu_ptr_[size_t(i) + 1]; ++t) acc -= lu_val_[size_t(t)] * y_[size_t(lu_col_[size_t(t)])];
            y_[size_t(i)] = acc / lu_val_[size_t(diag_[size_t(i)])];
        }
        x.resize(size_t(n));
        for (int j = 0; j < n; ++j) x[size_t(q_[size_t(j)])] = y_[size_t(j)];
    }

    bool solve_refined(const std::vector<double>& val, const std::vector<double>& rhs, std::vector<double>& x) {
        const int n = n_;
        apply(rhs, x);
        res_.resize(size_t(n));
        for (int round = 0; round < 4; ++round) {
            // Two measures per row. Componentwise: |b - A x|_i / (|b| + |A||x|)_i, what refinement normally reaches and the
            // stronger statement. Normwise: |b - A x|_i / (|b|_i + sum_k |a_ik| * max|x|), what Gaussian elimination
            // guarantees. A row that mixes coefficients of wildly different size (or whose terms have decayed into the
            // subnormal range, as at the far end of a long RC line) can be solved to rounding accuracy and still never meet
            // the first, so the solve is accepted when every row meets the first at 1e-10 or the second at 1e-13.
            double xmax = 0.0;
            for (int i = 0; i < n; ++i) xmax = std::max(xmax, std::fabs(x[size_t(i)]));
            if (!std::isfinite(xmax)) return false;
            double worst = 0.0, worst_loose = 0.0;  // over the rows: the measure each row does better on, scaled to its bound
            for (int r = 0; r < n; ++r) {
                double ax = 0.0, mag = std::fabs(rhs[size_t(r)]), rowsum = 0.0;
                for (int k = a_ptr_[size_t(r)]; k < a_ptr_[size_t(r) + 1]; ++k) {
                    const double t = val[size_t(k)] * x[size_t(a_col_[size_t(k)])];
                    ax += t;
                    mag += std::fabs(t);
                    rowsum += std::fabs(val[size_t(k)]);
                }
                const double res = rhs[size_t(r)] - ax;
                res_[size_t(r)] = res;
                if (!std::isfinite(res) || !std::isfinite(mag)) return false;  // an overflowed answer (std::max would skip a NaN)
                const double comp = mag > 0.0 ? std::fabs(res) / mag : 0.0;
                const double normw = std::fabs(rhs[size_t(r)]) + rowsum * (xmax + 1e-280);  // the floor: residuals down in the subnormal range are rounding noise
                const double norm = normw > 0.0 ? std::fabs(res) / normw : 0.0;
                worst = std::max(worst, std::min(comp / 1e-10, norm / 1e-13));
                worst_loose = std::max(worst_loose, std::min(comp / 1e-6, norm / 1e-10));
            }
            if (!(worst > 1.0)) return true;
            if (round == 3) return !(worst_loose > 1.0);
            ++stats.refinement_rounds;
            apply(res_, dx_);
            for (int i = 0; i < n; ++i) x[size_t(i)] += dx_[size_t(i)];
        }
        return true;
    }
};

}  // namespace nspice
