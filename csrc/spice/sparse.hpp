// Sparse linear algebra of the circuit simulator: CSR storage with a build-once pattern, a sparse LU
// with threshold partial pivoting, a Jacobi-preconditioned BiCGSTAB, and the solver facade.
//
// The reference keeps CSR only as a container and solves by densifying and running Gaussian
// elimination (nangila-spice/nangila-node/src/gpu_solver.rs:22-330); its GPU path is an SpMV, not a
// solve. Here the direct solve works on the sparse rows themselves (fill stays small for circuit
// matrices), and the Krylov solver is the host twin of the device solver built on the CSR SpMV
// kernel (csrc/kernels/spmv_csr.cu).
#pragma once
#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <map>
#include <string>
#include <numeric>
#include <stdexcept>
#include <utility>
#include <vector>

#include "sparse_lu.hpp"

namespace nspice {

struct CsrMatrix {
    int n = 0;
    std::vector<int> row_ptr{0};
    std::vector<int> col;
    std::vector<double> val;
    std::vector<double> rhs;
    std::vector<double> solution;

    CsrMatrix() = default;
    explicit CsrMatrix(int n_) : n(n_), row_ptr(size_t(n_) + 1, 0), rhs(size_t(n_), 0.0), solution(size_t(n_), 0.0) {}

    int nnz() const { return int(val.size()); }

    // Build from (row, col) -> value entries; duplicates are summed. Entries with |v| <= drop are
    // left out (drop < 0 keeps explicit zeros, which is what a reusable pattern wants).
    static CsrMatrix from_triplets(int n, const std::vector<std::tuple<int, int, double>>& t, double drop = -1.0) {
        std::vector<std::map<int, double>> rows(size_t(std::max(n, 0)));
        for (auto& e : t) {
            int r = std::get<0>(e), c = std::get<1>(e);
            if (r < 0 || c < 0 || r >= n || c >= n) throw std::out_of_range("triplet outside the matrix");
            rows[size_t(r)][c] += std::get<2>(e);
        }
        CsrMatrix m(n);
        for (int r = 0; r < n; ++r) {
            for (auto& kv : rows[size_t(r)])
                if (std::fabs(kv.second) > drop) { m.col.push_back(kv.first); m.val.push_back(kv.second); }
            m.row_ptr[size_t(r) + 1] = int(m.col.size());
        }
        return m;
    }
    static CsrMatrix from_dense(const std::vector<double>& a, int n, double drop) {
        CsrMatrix m(n);
        for (int r = 0; r < n; ++r) {
            for (int c = 0; c < n; ++c) {
                double v = a[size_t(r) * size_t(n) + size_t(c)];
                if (std::fabs(v) > drop) { m.col.push_back(c); m.val.push_back(v); }
            }
            m.row_ptr[size_t(r) + 1] = int(m.col.size());
        }
        return m;
    }
    std::vector<double> to_dense() const {
        std::vector<double> a(size_t(n) * size_t(n), 0.0);
        for (int r = 0; r < n; ++r)
            for (int k = row_ptr[size_t(r)]; k < row_ptr[size_t(r) + 1]; ++k) a[size_t(r) * size_t(n) + size_t(col[size_t(k)])] += val[size_t(k)];
        return a;
    }
    // Position of (r, c) in val, or -1.
    int slot(int r, int c) const {
        auto b = col.begin() + row_ptr[size_t(r)], e = col.begin() + row_ptr[size_t(r) + 1];
        auto it = std::lower_bound(b, e, c);
        return (it != e && *it == c) ? int(it - col.begin()) : -1;
    }
    void spmv(const double* x, double* y) const {
        for (int r = 0; r < n; ++r) {
            double acc = 0.0;
            for (int k = row_ptr[size_t(r)]; k < row_ptr[size_t(r) + 1]; ++k) acc += val[size_t(k)] * x[col[size_t(k)]];
            y[r] = acc;
        }
    }
    std::vector<double> spmv(const std::vector<double>& x) const {
        std::vector<double> y(size_t(n), 0.0);
        spmv(x.data(), y.data());
        return y;
    }
    double residual_inf(const std::vector<double>& x) const {
        std::vector<double> y = spmv(x);
        double m = 0.0;
        for (int i = 0; i < n; ++i) m = std::max(m, std::fabs(y[size_t(i)] - rhs[size_t(i)]));
        return m;
    }
};

// One-off solver (no state kept between calls); the transient loop uses FactoredLU (sparse_lu.hpp), which
// analyses a pattern once and refactors. This one stays as the fallback and as an independent check.
// Row-wise sparse Gaussian elimination on row-equilibrated data with threshold partial pivoting: among the rows whose entry
// in the pivot column is within a factor 10 of the largest, the shortest row wins (limits fill).
// One right-hand side is carried along, because a Newton iteration changes the matrix every solve.
inline bool sparse_lu_solve_once(const CsrMatrix& m, std::vector<double>& x) {
    const int n = m.n;
    using Row = std::vector<std::pair<int, double>>;
    std::vector<Row> rows(static_cast<size_t>(n));
    std::vector<double> b = m.rhs;
    b.resize(size_t(n), 0.0);
    std::vector<std::vector<int>> col_rows(static_cast<size_t>(n));
    for (int r = 0; r < n; ++r) {
        Row& row = rows[size_t(r)];
        for (int k = m.row_ptr[size_t(r)]; k < m.row_ptr[size_t(r) + 1]; ++k) {
            row.emplace_back(m.col[size_t(k)], m.val[size_t(k)]);
            col_rows[size_t(m.col[size_t(k)])].push_back(r);
        }
        // row equilibration: a row that pins a node with 1e12 S must not offer its 1e-3 S coupling
        // entry as a pivot, or the elimination loses every digit of the other rows
        double mx = 0.0;
        for (auto& e : row) mx = std::max(mx, std::fabs(e.second));
        if (mx > 0.0 && mx != 1.0) {
            for (auto& e : row) e.second /= mx;
            b[size_t(r)] /= mx;
        }
    }
    std::vector<int> pivot_row(size_t(n), -1);
    std::vector<char> used(size_t(n), 0);
    auto entry = [](const Row& row, int c) -> double {
        auto it = std::lower_bound(row.begin(), row.end(), c, [](const std::pair<int, double>& p, int cc) { return p.first < cc; });
        return (it != row.end() && it->first == c) ? it->second : 0.0;
    };
    Row merged;
    for (int k = 0; k < n; ++k) {
        double best = 0.0;
        auto& cands = col_rows[size_t(k)];
        std::sort(cands.begin(), cands.end());
        cands.erase(std::unique(cands.begin(), cands.end()), cands.end());
        for (int r : cands)
            if (!used[size_t(r)]) best = std::max(best, std::fabs(entry(rows[size_t(r)], k)));
        if (!(best > 1e-300)) return false;
        int p = -1;
        size_t plen = 0;
        for (int r : cands) {
            if (used[size_t(r)]) continue;
            double a = std::fabs(entry(rows[size_t(r)], k));
            if (a >= 0.1 * best && (p < 0 || rows[size_t(r)].size() < plen)) { p = r; plen = rows[size_t(r)].size(); }
        }
        used[size_t(p)] = 1;
        pivot_row[size_t(k)] = p;
        const Row& prow = rows[size_t(p)];
        const double pv = entry(prow, k);
        for (int r : cands) {
            if (used[size_t(r)]) continue;
            Row& row = rows[size_t(r)];
            double a = entry(row, k);
            if (a == 0.0) continue;
            const double f = a / pv;
            merged.clear();
            size_t i = 0, j = 0;
            while (i < row.size() || j < prow.size()) {
                if (j >= prow.size() || (i < row.size() && row[i].first < prow[j].first)) {
                    merged.push_back(row[i++]);
                } else if (i >= row.size() || prow[j].first < row[i].first) {
                    // fill-in; columns already eliminated cannot appear in a live pivot row
                    if (prow[j].first != k) { merged.emplace_back(prow[j].first, -f * prow[j].second); col_rows[size_t(prow[j].first)].push_back(r); }
                    ++j;
                } else {
                    if (row[i].first != k) merged.emplace_back(row[i].first, row[i].second - f * prow[j].second);
                    ++i; ++j;
                }
            }
            row.swap(merged);
            b[size_t(r)] -= f * b[size_t(p)];
        }
    }
    x.assign(size_t(n), 0.0);
    for (int k = n - 1; k >= 0; --k) {
        const Row& row = rows[size_t(pivot_row[size_t(k)])];
        double acc = b[size_t(pivot_row[size_t(k)])], pv = 0.0;
        for (auto& e : row) {
            if (e.first == k) pv = e.second;
            else if (e.first > k) acc -= e.second * x[size_t(e.first)];
        }
        x[size_t(k)] = acc / pv;
    }
    return true;
}

// The elimination above plus iterative refinement: while the componentwise backward error is above
// 1e-10 the residual system is solved again (at most three rounds). Circuit matrices pass at once;
// the refinement is for badly column-scaled systems.
inline bool sparse_lu_solve(const CsrMatrix& m, std::vector<double>& x) {
    if (!sparse_lu_solve_once(m, x)) return false;
    CsrMatrix res = m;
    std::vector<double> dx;
    for (int round = 0; round < 3; ++round) {
        double worst = 0.0;
        for (int r = 0; r < m.n; ++r) {
            double ax = 0.0, mag = std::fabs(m.rhs[size_t(r)]);
            for (int k = m.row_ptr[size_t(r)]; k < m.row_ptr[size_t(r) + 1]; ++k) {
                double t = m.val[size_t(k)] * x[size_t(m.col[size_t(k)])];
                ax += t;
                mag += std::fabs(t);
            }
            res.rhs[size_t(r)] = m.rhs[size_t(r)] - ax;
            if (mag > 0.0) worst = std::max(worst, std::fabs(res.rhs[size_t(r)]) / mag);
        }
        if (!(worst > 1e-10)) break;
        if (!sparse_lu_solve_once(res, dx)) break;
        for (int i = 0; i < m.n; ++i) x[size_t(i)] += dx[size_t(i)];
    }
    return true;
}

// Dense LU with partial pivoting; the oracle for the sparse paths.
inline bool dense_solve(std::vector<double> a, std::vector<double> b, int n, std::vector<double>& x) {
    for (int k = 0; k < n; ++k) {
        int p = k;
        for (int r = k + 1; r < n; ++r)
            if (std::fabs(a[size_t(r) * n + k]) > std::fabs(a[size_t(p) * n + k])) p = r;
        if (std::fabs(a[size_t(p) * n + k]) < 1e-300) return false;
        if (p != k) {
            for (int c = 0; c < n; ++c) std::swap(a[size_t(p) * n + c], a[size_t(k) * n + c]);
            std::swap(b[size_t(p)], b[size_t(k)]);
        }
        for (int r = k + 1; r < n; ++r) {
            double f = a[size_t(r) * n + k] / a[size_t(k) * n + k];
            if (f == 0.0) continue;
            for (int c = k; c < n; ++c) a[size_t(r) * n + c] -= f * a[size_t(k) * n + c];
            b[size_t(r)] -= f * b[size_t(k)];
        }
    }
    x.assign(size_t(n), 0.0);
    for (int k = n - 1; k >= 0; --k) {
        double acc = b[size_t(k)];
        for (int c = k + 1; c < n; ++c) acc -= a[size_t(k) * n + c] * x[size_t(c)];
        x[size_t(k)] = acc / a[size_t(k) * n + k];
    }
    return true;
}

struct KrylovResult { bool converged = false; int iterations = 0; double rel_residual = 0.0; };

// BiCGSTAB with a Jacobi (diagonal) preconditioner. `spmv` computes y = A x; passing the device
// SpMV here gives the GPU solve, passing CsrMatrix::spmv the host one.
template <class Spmv>
KrylovResult bicgstab(int n, Spmv&& spmv, const std::vector<double>& diag, const std::vector<double>& b,
                      std::vector<double>& x, double tol = 1e-10, int max_iter = 2000) {
    KrylovResult res;
    const size_t nn = size_t(n);
    std::vector<double> r(nn, 0.0), r0(nn, 0.0), p(nn, 0.0), v(nn, 0.0), s(nn, 0.0), t(nn, 0.0), ph(nn, 0.0), sh(nn, 0.0);
    x.resize(size_t(n), 0.0);
    auto dot = [&](const std::vector<double>& a, const std::vector<double>& c) { double s2 = 0; for (int i = 0; i < n; ++i) s2 += a[size_t(i)] * c[size_t(i)]; return s2; };
    auto inv = [&](int i) { double d = diag[size_t(i)]; return std::fabs(d) > 1e-300 ? 1.0 / d : 1.0; };
    spmv(x.data(), r.data());
    for (int i = 0; i < n; ++i) r[size_t(i)] = b[size_t(i)] - r[size_t(i)];
    r0 = r;
    double bnorm = std::sqrt(dot(b, b));
    if (bnorm == 0.0) bnorm = 1.0;
    double rho = 1, alpha = 1, omega = 1;
    res.rel_residual = std::sqrt(dot(r, r)) / bnorm;
    if (res.rel_residual < tol) { res.converged = true; return res; }
    for (int it = 1; it <= max_iter; ++it) {
        double rho_new = dot(r0, r);
        if (std::fabs(rho_new) < 1e-300) break;
        double beta = (rho_new / rho) * (alpha / omega);
        rho = rho_new;
        for (int i = 0; i < n; ++i) { p[size_t(i)] = r[size_t(i)] + beta * (p[size_t(i)] - omega * v[size_t(i)]); ph[size_t(i)] = p[size_t(i)] * inv(i); }
        spmv(ph.data(), v.data());
        double r0v = dot(r0, v);
        if (std::fabs(r0v) < 1e-300) break;
        alpha = rho / r0v;
        for (int i = 0; i < n; ++i) { s[size_t(i)] = r[size_t(i)] - alpha * v[size_t(i)]; sh[size_t(i)] = s[size_t(i)] * inv(i); }
        spmv(sh.data(), t.data());
        double tt = dot(t, t);
        omega = tt > 0 ? dot(t, s) / tt : 0.0;
        for (int i = 0; i < n; ++i) { x[size_t(i)] += alpha * ph[size_t(i)] + omega * sh[size_t(i)]; r[size_t(i)] = s[size_t(i)] - omega * t[size_t(i)]; }
        res.iterations = it;
        res.rel_residual = std::sqrt(dot(r, r)) / bnorm;
        if (res.rel_residual < tol) { res.converged = true; break; }
        if (omega == 0.0) break;
    }
    return res;
}

enum class LinearBackend { SparseLU, Dense, Krylov, Cuda };

// The device solver (FP64 CSR matrix resident on the GPU + BiCGSTAB, csrc/kernels/spmv_csr.cu) bound
// at run time with dlopen, so the simulator itself has no link-time CUDA dependency. The library is
// looked up at $NANGILA_KERNELS_LIB, else at the path given to set_library().
class CudaKrylov {
public:
    static std::string& library_path() { static std::string p; return p; }
    static void set_library(const std::string& p) { library_path() = p; }

    ~CudaKrylov() {
        if (ctx_ && destroy_) destroy_(ctx_);
        // the library stays loaded: unloading a CUDA library at exit is not worth the risk
    }
    bool available() {
        if (tried_) return create_ != nullptr;
        tried_ = true;
        const char* env = std::getenv("NANGILA_KERNELS_LIB");
        std::string path = env && *env ? env : library_path();
        if (path.empty()) return false;
        void* h = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
        if (!h) return false;
        create_ = reinterpret_cast<void* (*)()>(dlsym(h, "nangila_spmv_create"));
        destroy_ = reinterpret_cast<void (*)(void*)>(dlsym(h, "nangila_spmv_destroy"));
        load_ = reinterpret_cast<int (*)(void*, int, int, const int*, const int*, const double*)>(dlsym(h, "nangila_spmv_load"));
        update_ = reinterpret_cast<int (*)(void*, const double*)>(dlsym(h, "nangila_spmv_update_values"));
        solve_ = reinterpret_cast<int (*)(void*, const double*, double*, double, int, int*, double*)>(dlsym(h, "nangila_spmv_bicgstab"));
        if (!create_ || !destroy_ || !load_ || !update_ || !solve_) create_ = nullptr;
        return create_ != nullptr;
    }
    // Solves the row-equilibrated system; the pattern is uploaded once and only values afterwards.
    // Returns 0 = solved, 1 = did not converge, 2 = device error / library missing.
    int solve(const CsrMatrix& eq, std::vector<double>& x, double tol, int max_iter, int& iterations) {
        iterations = 0;
        if (!available()) return 2;
        if (!ctx_) ctx_ = create_();
        if (!ctx_) return 2;
        if (loaded_n_ != eq.n || loaded_nnz_ != eq.nnz() || pattern_ != eq.col || rows_ != eq.row_ptr) {
            if (load_(ctx_, eq.n, eq.nnz(), eq.row_ptr.data(), eq.col.data(), eq.val.data()) != 0) return 2;
            loaded_n_ = eq.n; loaded_nnz_ = eq.nnz(); pattern_ = eq.col; rows_ = eq.row_ptr;
        } else if (update_(ctx_, eq.val.data()) != 0) {
            return 2;
        }
        x.assign(size_t(eq.n), 0.0);
        double rel = 0.0;
        int rc = solve_(ctx_, eq.rhs.data(), x.data(), tol, max_iter, &iterations, &rel);
        return rc == 0 ? 0 : (rc == -1 ? 1 : 2);
    }
private:
    bool tried_ = false;
    void* ctx_ = nullptr;
    int loaded_n_ = -1, loaded_nnz_ = -1;
    std::vector<int> pattern_, rows_;
    void* (*create_)() = nullptr;
    void (*destroy_)(void*) = nullptr;
    int (*load_)(void*, int, int, const int*, const int*, const double*) = nullptr;
    int (*update_)(void*, const double*) = nullptr;
    int (*solve_)(void*, const double*, double*, double, int, int*, double*) = nullptr;
};

struct LinearSolverStats { uint64_t solves = 0, failures = 0, krylov_iterations = 0, krylov_fallbacks = 0, device_solves = 0, lu_fallbacks = 0; };

// Solver facade (the reference's GpuSolver::solve role): fills m.solution from m.rhs.
class LinearSolver {
public:
    LinearBackend backend = LinearBackend::SparseLU;
    LinearSolverStats stats;
    CudaKrylov cuda;
    FactoredLU lu;
    bool cuda_error = false;  // the device solver could not be loaded or reported a CUDA error; solves fell back to the sparse LU
    bool solve(CsrMatrix& m) {
        ++stats.solves;
        bool ok = false;
        if (backend == LinearBackend::Dense) {
            ok = dense_solve(m.to_dense(), m.rhs, m.n, m.solution);
        } else if (backend == LinearBackend::Krylov || backend == LinearBackend::Cuda) {
            // rows are equilibrated (divided by their largest entry) so that supply rows (entries of
            // 1) and stiff node rows (C / dt, ghost pins of 1e12) weigh the same in the residual norm
            CsrMatrix eq = m;
            for (int r = 0; r < m.n; ++r) {
                double mx = 0.0;
                for (int k = m.row_ptr[size_t(r)]; k < m.row_ptr[size_t(r) + 1]; ++k) mx = std::max(mx, std::fabs(m.val[size_t(k)]));
                if (mx > 0.0) {
                    for (int k = m.row_ptr[size_t(r)]; k < m.row_ptr[size_t(r) + 1]; ++k) eq.val[size_t(k)] /= mx;
                    eq.rhs[size_t(r)] /= mx;
                }
            }
            bool converged = false;
            if (backend == LinearBackend::Cuda) {
                int its = 0;
                int rc = cuda.solve(eq, m.solution, 1e-12, 4 * m.n + 50, its);
                stats.krylov_iterations += uint64_t(its);
                if (rc == 2) { cuda_error = true; converged = false; m.solution.assign(size_t(m.n), 0.0); }
                else { ++stats.device_solves; converged = rc == 0; }
            } else {
                std::vector<double> diag(size_t(m.n), 1.0);
                for (int r = 0; r < m.n; ++r) { int s = eq.slot(r, r); if (s >= 0 && std::fabs(eq.val[size_t(s)]) > 1e-3) diag[size_t(r)] = eq.val[size_t(s)]; }
                m.solution.assign(size_t(m.n), 0.0);
                KrylovResult kr = bicgstab(m.n, [&](const double* x, double* y) { eq.spmv(x, y); }, diag, eq.rhs, m.solution, 1e-12, 4 * m.n + 50);
                stats.krylov_iterations += uint64_t(kr.iterations);
                converged = kr.converged;
            }
            // accept only a small backward error: |A x - b|_i <= 1e-8 (|A||x| + |b|)_i + 1e-10 max|b| on the
            // equilibrated system (Newton itself stops at 1e-3 relative, so this is ample)
            ok = converged;
            double bmax = 0.0;
            for (double v : eq.rhs) bmax = std::max(bmax, std::fabs(v));
            for (int r = 0; ok && r < m.n; ++r) {
                double ax = 0.0, mag = std::fabs(eq.rhs[size_t(r)]);
                for (int k = eq.row_ptr[size_t(r)]; k < eq.row_ptr[size_t(r) + 1]; ++k) {
                    double t = eq.val[size_t(k)] * m.solution[size_t(eq.col[size_t(k)])];
                    ax += t;
                    mag += std::fabs(t);
                }
                if (!(std::fabs(ax - eq.rhs[size_t(r)]) <= 1e-8 * mag + 1e-10 * bmax + 1e-300)) ok = false;
            }
            if (!ok) { ++stats.krylov_fallbacks; ok = direct(m); }
        } else {
            ok = direct(m);
        }
        if (ok)
            for (double v : m.solution)
                if (!std::isfinite(v)) { ok = false; break; }
        if (!ok) ++stats.failures;
        return ok;
    }

private:
    bool direct(CsrMatrix& m) {
        if (lu.solve(m.n, m.row_ptr, m.col, m.val, m.rhs, m.solution)) return true;
        // Neither pivoting strategy gave a small backward error: the system is singular to working precision
        // (a DC iterate with chains of floating nets does that). Small systems get one more try with the one-off
        // elimination; large ones report the failure, which sends the DC solve to conductance stepping.
        if (m.n > 400) return false;
        ++stats.lu_fallbacks;
        return sparse_lu_solve(m, m.solution);
    }
};

}  // namespace nspice
