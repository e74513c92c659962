// Neighbour list of a periodic cubic box by a cell list, on the device.
//
// e3nn itself only ships an O(N^2) radius_graph (e3nn/nn/models/gate_points_2101.py:27-32) and states the
// periodic convention edge_vec = pos[src] - pos[dst] + shift
// (docs/guide/periodic_boundary_conditions.rst:134-136, gate_points_2101.py:328).  This builder produces,
// for every ordered pair with |pos[src] - pos[dst] + shift| <= cutoff (nearest image, src != dst), one
// edge; edges are sorted by destination, then by source, which is also the CSR order the fused
// convolution consumes (rowptr is an output).
//
// Integer work, HBM / latency bound, two passes because the edge count is not known in advance:
//   count: wrap positions into the box (fp64), bin atoms into cells of side box / floor(box / cutoff)
//          >= cutoff, exclusive scan of the cell counts, scatter atom indices into cell order, then one
//          thread per atom counts its neighbours in the 27 surrounding cells -> rowptr (exclusive scan);
//   fill:  the same walk writes (src, dst, shift) at rowptr[dst] + k and each thread sorts its own row
//          by source (rows have ~26 entries), which removes the scatter's dependence on atomics order:
//          the result is bit-identical from run to run.
// Distances are evaluated in fp64 as (p_j - p_i) + image, the same value with the opposite sign from
// either end of a pair, so the list is symmetric by construction.
#include "common.cuh"
#include "scan.cuh"

namespace e3b {
namespace {

struct NeighborScratch {
    double* p;            // [N,3] wrapped positions
    int32_t* cell_of;     // [N]
    int32_t* cell_count;  // [C]
    int32_t* cell_fill;   // [C]
    int64_t* cell_start;  // [C+1]
    int32_t* cell_atoms;  // [N]
    int32_t* deg;         // [N]
};

__host__ __device__ inline size_t align256(size_t x) { return (x + 255) & ~static_cast<size_t>(255); }

size_t neighbor_scratch_bytes(int64_t n, int64_t c) {
    return align256(sizeof(double) * 3 * n) + 3 * align256(sizeof(int32_t) * n) + 2 * align256(sizeof(int32_t) * c) +
           align256(sizeof(int64_t) * (c + 1));
}

NeighborScratch carve(void* scratch, int64_t n, int64_t c) {
    unsigned char* b = static_cast<unsigned char*>(scratch);
    NeighborScratch s;
    s.p = reinterpret_cast<double*>(b); b += align256(sizeof(double) * 3 * n);
    s.cell_of = reinterpret_cast<int32_t*>(b); b += align256(sizeof(int32_t) * n);
    s.cell_atoms = reinterpret_cast<int32_t*>(b); b += align256(sizeof(int32_t) * n);
    s.deg = reinterpret_cast<int32_t*>(b); b += align256(sizeof(int32_t) * n);
    s.cell_count = reinterpret_cast<int32_t*>(b); b += align256(sizeof(int32_t) * c);
    s.cell_fill = reinterpret_cast<int32_t*>(b); b += align256(sizeof(int32_t) * c);
    s.cell_start = reinterpret_cast<int64_t*>(b);
    return s;
}

__global__ void wrap_bin_kernel(const float* __restrict__ pos, int64_t n, double box, int nc, double* __restrict__ p,
                                int32_t* __restrict__ cell_of, int32_t* __restrict__ cell_count) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int c[3];
#pragma unroll
    for (int a = 0; a < 3; ++a) {
        const double x = static_cast<double>(pos[i * 3 + a]);
        double w = x - floor(x / box) * box;
        if (w >= box) w -= box;
        if (w < 0.0) w = 0.0;
        p[i * 3 + a] = w;
        int q = static_cast<int>(w / box * nc);
        c[a] = q < 0 ? 0 : (q >= nc ? nc - 1 : q);
    }
    const int cell = (c[0] * nc + c[1]) * nc + c[2];
    cell_of[i] = cell;
    atomicAdd(cell_count + cell, 1);
}

__global__ void cell_scatter_kernel(const int32_t* __restrict__ cell_of, int64_t n, const int64_t* __restrict__ cell_start,
                                    int32_t* __restrict__ cell_fill, int32_t* __restrict__ cell_atoms) {
    const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int cell = cell_of[i];
    const int slot = atomicAdd(cell_fill + cell, 1);
    cell_atoms[cell_start[cell] + slot] = static_cast<int32_t>(i);
}

// One thread per destination atom i of the rows [row0, row0 + nrows).  FILL == false: deg[i - row0] = number of
// neighbours.  FILL == true: writes the row's edges at rowptr[i - row0] and sorts them by source.
template <bool FILL>
__global__ void neighbor_walk_kernel(const float* __restrict__ pos, const double* __restrict__ p, const int32_t* __restrict__ cell_of,
                                     const int64_t* __restrict__ cell_start, const int32_t* __restrict__ cell_atoms, int64_t row0,
                                     int64_t nrows, double box, double cutoff2, int nc, int32_t* __restrict__ deg,
                                     const int64_t* __restrict__ rowptr, int64_t* __restrict__ edge_src,
                                     int64_t* __restrict__ edge_dst, float* __restrict__ shift) {
    const int64_t local = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (local >= nrows) return;
    const int64_t i = row0 + local;
    const double pix = p[i * 3], piy = p[i * 3 + 1], piz = p[i * 3 + 2];
    const int cell = cell_of[i];
    const int cz = cell % nc, cy = (cell / nc) % nc, cx = cell / (nc * nc);
    // offset between the caller's coordinates and the wrapped ones (0 for atoms inside the box)
    const double oix = pix - static_cast<double>(pos[i * 3]), oiy = piy - static_cast<double>(pos[i * 3 + 1]),
                 oiz = piz - static_cast<double>(pos[i * 3 + 2]);
    const int64_t base = FILL ? rowptr[local] : 0;
    int count = 0;
    for (int dx = -1; dx <= 1; ++dx) {
        int nx = cx + dx;
        double sx = 0.0;
        if (nx < 0) { nx += nc; sx = -box; } else if (nx >= nc) { nx -= nc; sx = box; }
        for (int dy = -1; dy <= 1; ++dy) {
            int ny = cy + dy;
            double sy = 0.0;
            if (ny < 0) { ny += nc; sy = -box; } else if (ny >= nc) { ny -= nc; sy = box; }
            for (int dz = -1; dz <= 1; ++dz) {
                int nz = cz + dz;
                double sz = 0.0;
                if (nz < 0) { nz += nc; sz = -box; } else if (nz >= nc) { nz -= nc; sz = box; }
                const int ncell = (nx * nc + ny) * nc + nz;
                const int64_t a0 = cell_start[ncell], a1 = cell_start[ncell + 1];
                for (int64_t a = a0; a < a1; ++a) {
                    const int j = cell_atoms[a];
                    if (j == i) continue;
                    const double ddx = (p[j * 3] - pix) + sx, ddy = (p[j * 3 + 1] - piy) + sy, ddz = (p[j * 3 + 2] - piz) + sz;
                    if (ddx * ddx + ddy * ddy + ddz * ddz <= cutoff2) {
                        if (FILL) {
                            const int64_t e = base + count;
                            edge_src[e] = j;
                            edge_dst[e] = i;
                            // edge_vec = pos[src] - pos[dst] + shift must equal (p_j - p_i) + image
                            shift[e * 3] = static_cast<float>((p[j * 3] - static_cast<double>(pos[j * 3])) - oix + sx);
                            shift[e * 3 + 1] = static_cast<float>((p[j * 3 + 1] - static_cast<double>(pos[j * 3 + 1])) - oiy + sy);
                            shift[e * 3 + 2] = static_cast<float>((p[j * 3 + 2] - static_cast<double>(pos[j * 3 + 2])) - oiz + sz);
                        }
                        ++count;
                    }
                }
            }
        }
    }
    if (!FILL) {
        deg[local] = count;
        return;
    }
    // insertion sort of this row by source index (rows are short; the row is private to this thread)
    for (int a = 1; a < count; ++a) {
        const int64_t ea = base + a;
        const int64_t key = edge_src[ea];
        const float s0 = shift[ea * 3], s1 = shift[ea * 3 + 1], s2 = shift[ea * 3 + 2];
        int64_t b = ea - 1;
        while (b >= base && edge_src[b] > key) {
            edge_src[b + 1] = edge_src[b];
            shift[(b + 1) * 3] = shift[b * 3]; shift[(b + 1) * 3 + 1] = shift[b * 3 + 1]; shift[(b + 1) * 3 + 2] = shift[b * 3 + 2];
            --b;
        }
        edge_src[b + 1] = key;
        shift[(b + 1) * 3] = s0; shift[(b + 1) * 3 + 1] = s1; shift[(b + 1) * 3 + 2] = s2;
    }
}

int cells_per_side(double box, double cutoff) {
    const double q = floor(box / cutoff);
    return q > 1024.0 ? 1024 : static_cast<int>(q);   // more cells than that only lengthens the scan
}

int check_rows(int64_t n, int64_t row0, int64_t row1) {
    if (row0 < 0 || row1 < row0 || row1 > n) return fail(E3B_ERR_ARG, "neighbor list: rows [%lld, %lld) outside [0, %lld)",
                                                          static_cast<long long>(row0), static_cast<long long>(row1), static_cast<long long>(n));
    return E3B_OK;
}

int check_neighbor_args(int64_t n, double box, double cutoff) {
    if (n < 0) return fail(E3B_ERR_ARG, "neighbor list: negative atom count");
    if (n > 2147483647LL) return fail(E3B_ERR_ARG, "neighbor list: more than 2^31 - 1 atoms");
    if (!(cutoff > 0.0) || !(box > 0.0)) return fail(E3B_ERR_ARG, "neighbor list: box and cutoff must be positive");
    if (box < 3.0 * cutoff)
        return fail(E3B_ERR_UNSUPPORTED, "neighbor list: the cell list needs box >= 3 x cutoff (box %g, cutoff %g)", box, cutoff);
    return E3B_OK;
}

}  // namespace
}  // namespace e3b

extern "C" int64_t e3b_neighbor_scratch_bytes(int64_t num_atoms, double box, double cutoff) {
    using namespace e3b;
    if (num_atoms < 0 || !(cutoff > 0.0) || box < 3.0 * cutoff) return -1;
    const int64_t nc = cells_per_side(box, cutoff);
    return static_cast<int64_t>(neighbor_scratch_bytes(num_atoms, nc * nc * nc));
}

extern "C" int e3b_neighbor_count(const float* pos, int64_t num_atoms, double box, double cutoff, void* scratch,
                                  int64_t scratch_bytes, int64_t* rowptr, void* stream) {
    return e3b_neighbor_count_rows(pos, num_atoms, box, cutoff, scratch, scratch_bytes, 0, num_atoms, rowptr, stream);
}

extern "C" int e3b_neighbor_count_rows(const float* pos, int64_t num_atoms, double box, double cutoff, void* scratch,
                                       int64_t scratch_bytes, int64_t row0, int64_t row1, int64_t* rowptr, void* stream) {
    using namespace e3b;
    if (int rc = check_neighbor_args(num_atoms, box, cutoff)) return rc;
    if (int rc = check_rows(num_atoms, row0, row1)) return rc;
    if (!rowptr) return fail(E3B_ERR_ARG, "neighbor_count: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t nrows = row1 - row0;
    if (num_atoms == 0 || nrows == 0) {
        E3B_CUDA_TRY(cudaMemsetAsync(rowptr, 0, sizeof(int64_t), s));
        return E3B_OK;
    }
    const int nc = cells_per_side(box, cutoff);
    const int64_t cells = static_cast<int64_t>(nc) * nc * nc;
    if (!pos || !scratch) return fail(E3B_ERR_ARG, "neighbor_count: null pointer");
    if (scratch_bytes < static_cast<int64_t>(neighbor_scratch_bytes(num_atoms, cells)) || reinterpret_cast<uintptr_t>(scratch) % 256 != 0)
        return fail(E3B_ERR_ARG, "neighbor_count: scratch too small or not 256-byte aligned");
    NeighborScratch sc = carve(scratch, num_atoms, cells);
    E3B_CUDA_TRY(cudaMemsetAsync(sc.cell_count, 0, sizeof(int32_t) * cells, s));
    E3B_CUDA_TRY(cudaMemsetAsync(sc.cell_fill, 0, sizeof(int32_t) * cells, s));
    const int threads = 256;
    const unsigned grid = static_cast<unsigned>(ceil_div(num_atoms, threads));
    wrap_bin_kernel<<<grid, threads, 0, s>>>(pos, num_atoms, box, nc, sc.p, sc.cell_of, sc.cell_count);
    exclusive_scan_i32_kernel<<<1, 1024, 0, s>>>(sc.cell_count, cells, sc.cell_start);
    cell_scatter_kernel<<<grid, threads, 0, s>>>(sc.cell_of, num_atoms, sc.cell_start, sc.cell_fill, sc.cell_atoms);
    const unsigned row_grid = static_cast<unsigned>(ceil_div(nrows, threads));
    neighbor_walk_kernel<false><<<row_grid, threads, 0, s>>>(pos, sc.p, sc.cell_of, sc.cell_start, sc.cell_atoms, row0, nrows, box,
                                                             cutoff * cutoff, nc, sc.deg, nullptr, nullptr, nullptr, nullptr);
    exclusive_scan_i32_kernel<<<1, 1024, 0, s>>>(sc.deg, nrows, rowptr);
    return check_launch("neighbor_count");
}

extern "C" int e3b_neighbor_fill(const float* pos, int64_t num_atoms, double box, double cutoff, void* scratch,
                                 int64_t scratch_bytes, const int64_t* rowptr, int64_t* edge_src, int64_t* edge_dst,
                                 float* shift, void* stream) {
    return e3b_neighbor_fill_rows(pos, num_atoms, box, cutoff, scratch, scratch_bytes, 0, num_atoms, rowptr, edge_src, edge_dst,
                                  shift, stream);
}

extern "C" int e3b_neighbor_fill_rows(const float* pos, int64_t num_atoms, double box, double cutoff, void* scratch,
                                      int64_t scratch_bytes, int64_t row0, int64_t row1, const int64_t* rowptr, int64_t* edge_src,
                                      int64_t* edge_dst, float* shift, void* stream) {
    using namespace e3b;
    if (int rc = check_neighbor_args(num_atoms, box, cutoff)) return rc;
    if (int rc = check_rows(num_atoms, row0, row1)) return rc;
    const int64_t nrows = row1 - row0;
    if (num_atoms == 0 || nrows == 0) return E3B_OK;
    const int nc = cells_per_side(box, cutoff);
    const int64_t cells = static_cast<int64_t>(nc) * nc * nc;
    if (!pos || !scratch || !rowptr || !edge_src || !edge_dst || !shift) return fail(E3B_ERR_ARG, "neighbor_fill: null pointer");
    if (scratch_bytes < static_cast<int64_t>(neighbor_scratch_bytes(num_atoms, cells)) || reinterpret_cast<uintptr_t>(scratch) % 256 != 0)
        return fail(E3B_ERR_ARG, "neighbor_fill: scratch too small or not 256-byte aligned");
    NeighborScratch sc = carve(scratch, num_atoms, cells);
    const int threads = 256;
    const unsigned grid = static_cast<unsigned>(ceil_div(nrows, threads));
    neighbor_walk_kernel<true><<<grid, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        pos, sc.p, sc.cell_of, sc.cell_start, sc.cell_atoms, row0, nrows, box, cutoff * cutoff, nc, sc.deg, rowptr, edge_src,
        edge_dst, shift);
    return check_launch("neighbor_fill");
}
