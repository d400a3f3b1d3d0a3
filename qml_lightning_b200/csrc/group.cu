// Element grouping of atoms: a deterministic, sync-free counting sort on the device.
//
// The upstream model loops over elements on the host and gathers the atoms of each element with boolean masks and
// torch.where (models/hadamard_features.py:99-107), which costs a device-to-host synchronisation per element.
// Here three small kernels build the permutation once per batch:
//   1. count   : per block of GROUP_MOLS molecules, number of atoms of each model element
//   2. scan    : exclusive prefix over the blocks per element; groups are padded to QMLB_ROW_TILE rows
//   3. assign  : every block re-walks its molecules in (molecule, atom) order and hands out rows
// The row order inside a group therefore follows (molecule, atom) order and never depends on scheduling.
#include "common.cuh"

namespace {

constexpr int GROUP_MOLS = 32;     // molecules per block (one warp per block)
constexpr int MAX_ELEMENTS = 32;

__device__ __forceinline__ int element_of(float z, const float *elements, int nel) {
    const float q = (float)(int)z;
    int idx = -1;
    for (int j = 0; j < nel; ++j)
        if (q == elements[j]) idx = j;
    return idx;
}

__global__ void count_kernel(const float *__restrict__ Z, const int *__restrict__ counts,
                             const float *__restrict__ elements, int nel, int nb, int A, int *__restrict__ block_counts) {
    const int lane = threadIdx.x;
    const int m0 = blockIdx.x * GROUP_MOLS;
    const int m1 = min(nb, m0 + GROUP_MOLS);
    int local[MAX_ELEMENTS];
    for (int e = 0; e < nel; ++e) local[e] = 0;
    const long s0 = (long)m0 * A, s1 = (long)m1 * A;
    for (long s = s0 + lane; s < s1; s += 32) {
        const int m = (int)(s / A), a = (int)(s % A);
        if (a < counts[m]) {
            const int e = element_of(Z[s], elements, nel);
            for (int q = 0; q < nel; ++q) local[q] += (q == e);
        }
    }
    for (int e = 0; e < nel; ++e) {
        int v = local[e];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(QMLB_FULL_MASK, v, o);
        if (lane == 0) block_counts[(size_t)e * gridDim.x + blockIdx.x] = v;
    }
}

// One block; block_counts[e][blk] -> exclusive prefix in place; group_start[e] with tile padding.
__global__ void scan_kernel(int *__restrict__ block_counts, int nblocks, int nel, int *__restrict__ group_start) {
    __shared__ int warp_tot[32];
    __shared__ int carry;
    __shared__ int totals[MAX_ELEMENTS + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int e = 0; e < nel; ++e) {
        if (threadIdx.x == 0) carry = 0;
        __syncthreads();
        int *col = block_counts + (size_t)e * nblocks;
        for (int base = 0; base < nblocks; base += blockDim.x) {
            const int idx = base + threadIdx.x;
            const int v = idx < nblocks ? col[idx] : 0;
            int inc = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(QMLB_FULL_MASK, inc, o);
                if (lane >= o) inc += t;
            }
            if (lane == 31) warp_tot[warp] = inc;
            __syncthreads();
            int woff = 0;
            for (int w = 0; w < warp; ++w) woff += warp_tot[w];
            int chunk_total = 0;
            for (int w = 0; w < nwarps; ++w) chunk_total += warp_tot[w];
            if (idx < nblocks) col[idx] = carry + woff + inc - v;
            __syncthreads();
            if (threadIdx.x == 0) carry += chunk_total;
            __syncthreads();
        }
        if (threadIdx.x == 0) totals[e] = carry;
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        int start = 0;
        for (int e = 0; e < nel; ++e) {
            group_start[e] = start;
            start += (totals[e] + QMLB_ROW_TILE - 1) / QMLB_ROW_TILE * QMLB_ROW_TILE;
        }
        group_start[nel] = start;
    }
}

__global__ void assign_kernel(const float *__restrict__ Z, const int *__restrict__ counts,
                              const float *__restrict__ elements, int nel, int nb, int A,
                              const int *__restrict__ block_base, const int *__restrict__ group_start,
                              int *__restrict__ row_of_slot, int *__restrict__ slot_of_row, long rows_cap) {
    const int lane = threadIdx.x;
    const int m0 = blockIdx.x * GROUP_MOLS;
    const int m1 = min(nb, m0 + GROUP_MOLS);
    int next[MAX_ELEMENTS];
    for (int e = 0; e < nel; ++e) next[e] = group_start[e] + block_base[(size_t)e * gridDim.x + blockIdx.x];
    const long s0 = (long)m0 * A, s1 = (long)m1 * A;
    for (long sb = s0; sb < s1; sb += 32) {
        const long s = sb + lane;
        int e = -1;
        if (s < s1) {
            const int m = (int)(s / A), a = (int)(s % A);
            if (a < counts[m]) e = element_of(Z[s], elements, nel);
        }
        int row = -1;
        for (int q = 0; q < nel; ++q) {
            const unsigned msk = __ballot_sync(QMLB_FULL_MASK, e == q);
            if (e == q) row = next[q] + __popc(msk & ((1u << lane) - 1u));
            next[q] += __popc(msk);
        }
        if (s < s1) {
            // a row capacity below the real atom count cannot be seen by the host without a synchronisation: such atoms
            // are marked, and the kernels that produce energies and gradients turn the mark into NaN for their molecule
            if (row >= rows_cap) row = QMLB_ROW_OVERFLOW;
            row_of_slot[s] = row;
            if (row >= 0) slot_of_row[row] = (int)s;
        }
    }
}

// Small batches (at most SMALL_MOLS molecules): the three steps in ONE launch of one block.  Warp w owns the molecules
// [32 w, 32 w + 32) exactly like block w of the three-kernel path, so both paths produce the same permutation; the
// per-warp counts and their prefix stay in shared memory.  Saves two launches and the memset node, which is what a
// 1,000-molecule prediction step is made of.
constexpr int SMALL_MOLS = 1024;
__global__ void __launch_bounds__(1024)
group_small_kernel(const float *__restrict__ Z, const int *__restrict__ counts, const float *__restrict__ elements, int nel,
                   int nb, int A, int *__restrict__ row_of_slot, int *__restrict__ slot_of_row, int *__restrict__ group_start,
                   long rows_cap) {
    __shared__ int cnt[MAX_ELEMENTS][32];      // [element][warp] counts, then exclusive prefix over the warps
    __shared__ int gstart[MAX_ELEMENTS + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (long r = threadIdx.x; r < rows_cap; r += blockDim.x) slot_of_row[r] = -1;
    const int m0 = warp * GROUP_MOLS, m1 = min(nb, m0 + GROUP_MOLS);
    const long s0 = (long)m0 * A, s1 = (long)max(m1, m0) * A;
    int local[MAX_ELEMENTS];
    for (int e = 0; e < nel; ++e) local[e] = 0;
    for (long s = s0 + lane; s < s1; s += 32) {
        const int m = (int)(s / A), a = (int)(s % A);
        if (a < counts[m]) {
            const int e = element_of(Z[s], elements, nel);
            for (int q = 0; q < nel; ++q) local[q] += (q == e);
        }
    }
    for (int e = 0; e < nel; ++e) {
        int v = local[e];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(QMLB_FULL_MASK, v, o);
        if (lane == 0) cnt[e][warp] = v;
    }
    __syncthreads();
    if (warp < nel) {                            // warp e scans element e over the 32 owning warps
        const int v = cnt[warp][lane];
        int inc = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(QMLB_FULL_MASK, inc, o);
            if (lane >= o) inc += t;
        }
        cnt[warp][lane] = inc - v;
        if (lane == 31) gstart[warp + 1] = (inc + QMLB_ROW_TILE - 1) / QMLB_ROW_TILE * QMLB_ROW_TILE;   // padded size
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int start = 0;
        for (int e = 0; e < nel; ++e) {
            const int padded = gstart[e + 1];
            gstart[e] = start;
            group_start[e] = start;
            start += padded;
        }
        gstart[nel] = start;
        group_start[nel] = start;
    }
    __syncthreads();
    int next[MAX_ELEMENTS];
    for (int e = 0; e < nel; ++e) next[e] = gstart[e] + cnt[e][warp];
    for (long sb = s0; sb < s1; sb += 32) {
        const long s = sb + lane;
        int e = -1;
        if (s < s1) {
            const int m = (int)(s / A), a = (int)(s % A);
            if (a < counts[m]) e = element_of(Z[s], elements, nel);
        }
        int row = -1;
        for (int q = 0; q < nel; ++q) {
            const unsigned msk = __ballot_sync(QMLB_FULL_MASK, e == q);
            if (e == q) row = next[q] + __popc(msk & ((1u << lane) - 1u));
            next[q] += __popc(msk);
        }
        if (s < s1) {
            if (row >= rows_cap) row = QMLB_ROW_OVERFLOW;
            row_of_slot[s] = row;
            if (row >= 0) slot_of_row[row] = (int)s;
        }
    }
}

}  // namespace

extern "C" size_t qmlb_rows_capacity(size_t n_atoms_upper, int nelements) {
    const size_t cap = n_atoms_upper + (size_t)nelements * (QMLB_ROW_TILE - 1);
    return (cap + QMLB_ROW_TILE - 1) / QMLB_ROW_TILE * QMLB_ROW_TILE;
}

extern "C" size_t qmlb_group_scratch_bytes(int nb, int nelements) {
    const size_t nblocks = ((size_t)nb + GROUP_MOLS - 1) / GROUP_MOLS;
    return sizeof(int) * nblocks * (size_t)nelements + 256;
}

extern "C" int qmlb_group_by_element(const float *Z, const int *atom_counts, const float *elements, int nelements,
                                     int nb, int A, int *row_of_slot, int *slot_of_row, int *group_start,
                                     size_t rows_cap, void *scratch, qmlb_stream_t stream) {
    QMLB_REQUIRE(Z && atom_counts && elements && row_of_slot && slot_of_row && group_start && scratch,
                 "qmlb_group_by_element: null tensor");
    QMLB_REQUIRE(nelements > 0 && nelements <= MAX_ELEMENTS, "qmlb_group_by_element: 1..%d elements supported", MAX_ELEMENTS);
    QMLB_REQUIRE(nb > 0 && A > 0, "qmlb_group_by_element: bad batch shape");
    QMLB_REQUIRE((size_t)nb * A < (size_t)1 << 31, "qmlb_group_by_element: nb*A must fit in int32");
    QMLB_REQUIRE(rows_cap % QMLB_ROW_TILE == 0 && rows_cap < (size_t)1 << 31, "qmlb_group_by_element: bad rows_cap");
    cudaStream_t st = qmlb::as_stream(stream);
    if (nb <= SMALL_MOLS) {
        group_small_kernel<<<1, 1024, 0, st>>>(Z, atom_counts, elements, nelements, nb, A, row_of_slot, slot_of_row, group_start,
                                               (long)rows_cap);
        return qmlb::check_launch("qmlb_group_by_element");
    }
    const int nblocks = (nb + GROUP_MOLS - 1) / GROUP_MOLS;
    int *block_counts = static_cast<int *>(scratch);
    // padding rows carry no atom: all bytes 0xFF = -1
    if (cudaMemsetAsync(slot_of_row, 0xFF, rows_cap * sizeof(int), st) != cudaSuccess)
        return qmlb::check_launch("qmlb_group_by_element(memset)");
    count_kernel<<<nblocks, 32, 0, st>>>(Z, atom_counts, elements, nelements, nb, A, block_counts);
    scan_kernel<<<1, 1024, 0, st>>>(block_counts, nblocks, nelements, group_start);
    assign_kernel<<<nblocks, 32, 0, st>>>(Z, atom_counts, elements, nelements, nb, A, block_counts, group_start,
                                          row_of_slot, slot_of_row, (long)rows_cap);
    return qmlb::check_launch("qmlb_group_by_element");
}

// ---- allocation-free variant ---------------------------------------------------------------------------------
// Same grouping, but the per-block counters live in a fixed array inside the library image instead of in memory
// the caller allocated.  It serves callers that are handed their input and output buffers and may not allocate:
// a force-field plug-in called back by a simulation engine that owns the whole device-memory budget, or a
// service thread that must never enter the allocator because cudaMalloc / cudaFree serialise against every
// stream of the process.
namespace {

// Held by every GPU that loads the library until the process exits (QMLB_GROUP_STATIC_SCRATCH_BYTES = 1 MiB).
static __device__ __align__(256) unsigned char g_group_scratch[QMLB_GROUP_STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
void *g_group_scratch_addr[MAX_DEVICES] = {};  // device address of the array, per device ordinal

// In host code `g_group_scratch` is only a handle of the symbol, not an address a kernel could use: the device
// address has to be looked up, with the device current, through cudaGetSymbolAddress.  Done once per device.
int static_scratch_address(void **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        qmlb::set_error("qmlb_group_by_element_noalloc: cudaGetDevice: %s (device %d)", cudaGetErrorString(e), dev);
        return QMLB_ERR_CUDA;
    }
    void *p = __atomic_load_n(&g_group_scratch_addr[dev], __ATOMIC_ACQUIRE);
    if (p == nullptr) {
        e = cudaGetSymbolAddress(&p, g_group_scratch);
        if (e != cudaSuccess || p == nullptr) {
            qmlb::set_error("qmlb_group_by_element_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            return QMLB_ERR_CUDA;
        }
        __atomic_store_n(&g_group_scratch_addr[dev], p, __ATOMIC_RELEASE);  // every thread would store the same value
    }
    *out = p;
    return QMLB_OK;
}

}  // namespace

extern "C" int qmlb_group_by_element_noalloc(const float *Z, const int *atom_counts, const float *elements,
                                             int nelements, int nb, int A, int *row_of_slot, int *slot_of_row,
                                             int *group_start, size_t rows_cap, qmlb_stream_t stream) {
    QMLB_REQUIRE(nb > 0 && nelements > 0, "qmlb_group_by_element_noalloc: bad batch shape");
    const size_t need = qmlb_group_scratch_bytes(nb, nelements);
    QMLB_REQUIRE(need <= (size_t)QMLB_GROUP_STATIC_SCRATCH_BYTES,
                 "qmlb_group_by_element_noalloc: nb=%d molecules with %d elements need %zu bytes of scratch, the built-in "
                 "array holds %u; split the batch or use qmlb_group_by_element with caller-owned scratch",
                 nb, nelements, need, (unsigned)QMLB_GROUP_STATIC_SCRATCH_BYTES);
    void *scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    // Nothing in the array has to start at zero: the counting kernel overwrites every counter that the scan and
    // the assignment read, so contents left by an earlier call are never observed.
    return qmlb_group_by_element(Z, atom_counts, elements, nelements, nb, A, row_of_slot, slot_of_row, group_start,
                                 rows_cap, scratch, stream);
}
