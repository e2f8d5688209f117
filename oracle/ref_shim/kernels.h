/* TEST INFRASTRUCTURE ONLY.
 *
 * Hand-written stand-in for the header the reference's code generator would
 * emit (python/kernel_gen.py:421-465 writes include/kernels.h; python/grid_gen.py:19-42
 * prepends a `grid_dims` table to include/tiling.h).  It lets the reference's
 * checked-in sources compile where they lie, without running any generator:
 * it only DECLARES what src/kernels/haswell/dense.cpp:8 already defines and
 * provides the two lookup objects the sources index.
 */
#pragma once

#define MR_FACT 2
#define NR_FACT 16
#define MR_MIN 6
#define NR_MIN 16

typedef void ref_shim_ukernel_t(float* A, float* B, float* C, int m, int n, int k);

/* defined by the reference in src/kernels/haswell/dense.cpp:8 */
void cake_sgemm_haswell_6x16(float* A, float* B, float* C, int m, int n, int k);

/* src/cake_sgemm_k_first.cpp:121 calls kernel_map[m_map][n_map]; with the one
 * checked-in register tile (6x16) both indices are 0. */
static ref_shim_ukernel_t* kernel_map[1][1] = {{cake_sgemm_haswell_6x16}};

/* src/block_sizing.cpp:613-625 reads grid_dims[ncores - p][i] == "(i+1) divides p".
 * The generated table bakes in the build host's core count; this object
 * answers the same question for whatever core count the driver announces. */
extern int ref_shim_ncores;
struct ref_shim_grid_row {
    int p;
    bool operator[](int i) const { return p > 0 && (p % (i + 1)) == 0; }
};
struct ref_shim_grid {
    ref_shim_grid_row operator[](int r) const { return ref_shim_grid_row{ref_shim_ncores - r}; }
};
static const ref_shim_grid grid_dims = {};
