/* grace_b200 - C ABI of the B200-native GRACE evaluation backend (libgrace_b200.so).
 *
 * Every entry point replaces one member of the reference's GPU backend interface `namespace grace_runtime_kk`
 * (python/kk/kk_api.h:14-156, "ABI 7"), which the reference binds to Python in python/kk/kk_module.cpp:200-275.
 * Argument meaning, array conventions and error classes are the reference's:
 *   - atom types are 1-based indices into the species list given at create time;
 *   - positions [n][3] and cell [3][3] (rows = cell vectors, full rank; open directions padded by the caller) are
 *     fp64; pbc is one byte per direction;
 *   - forces [n][3] in the caller's atom order; virial[6] = sum over bonds (x_i - x_j) (x) f_i in the order
 *     xx yy zz xy xz yz; stress = -virial[[0,1,2,5,4,3]] / V is left to the caller as in the reference
 *     (python/grace_runtime/calculator.py:155-157);
 *   - outputs are written, never accumulated; the caller owns inputs and outputs.
 * Functions return a status: 0 ok, 1 invalid argument (reference: std::invalid_argument / ValueError), 2 runtime or
 * device error (std::runtime_error), 3 out of device memory, 4 unsupported model or feature.  The message of the last
 * failure of the calling thread is grace_last_error().  Nothing here aborts or traps.  All device work of a process
 * is serialised internally (kk_core.cpp:58-63, 805-806), so any host thread may call.
 * There is no CPU fallback: every compute call runs the CUDA kernels of this library on the initialised device.
 */
#ifndef GRACE_B200_H
#define GRACE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)    /* the library is built with hidden visibility: only this ABI is exported */
#endif

#define GRACE_OK 0
#define GRACE_INVALID_ARGUMENT 1
#define GRACE_RUNTIME_ERROR 2
#define GRACE_OUT_OF_MEMORY 3
#define GRACE_UNSUPPORTED 4

/* the integer the Python side compares with its own (python/grace_runtime/_gpu.py:18) */
#define GRACE_B200_ABI 7

/* compute flags (kk_api.h:84-86: energies, uq, energy_only) */
#define GRACE_FLAG_ENERGIES 1     /* also write per-atom energies */
#define GRACE_FLAG_ENERGY_ONLY 2  /* no reverse pass: forces and virial are not written */
#define GRACE_FLAG_UQ 4           /* also the UQ outputs (gamma, sigma, cluster per atom) where grace_*_set_uq_outputs put them */

typedef struct grace_model grace_model;
typedef struct grace_system grace_system;
typedef struct grace_batch grace_batch;

/* ---- process / device (kk_api.h:16-33) ---- */
int grace_initialize(int device);              /* initialize(device): one GPU per process */
int grace_finalize(void);                      /* finalize(): releases the device buffers of every live object */
int grace_initialized(void);                   /* initialized() */
int grace_device(void);                        /* device() */
const char *grace_arch(void);                  /* arch(): "sm100" */
const char *grace_platform(void);              /* platform(): "cuda" */
const char *grace_blas(void);                  /* blas(): "" (no GEMM library on the path) */
int grace_abi(void);                           /* the module attribute ABI */
int grace_memory_info(size_t *free_bytes, size_t *total_bytes);   /* memory_info() */
/* tests: the nth device allocation from now on whose label contains `label` fails as out of memory (nth <= 0: off) */
int grace_debug_fail_alloc(const char *label, int nth);           /* debug_fail_alloc(label, nth) */
/* tests: the nth kernel launch check from now on reports an out-of-memory launch (0: off) */
int grace_debug_fail_launch(int nth);                             /* debug_fail_launch(nth) */
/* Microbenchmarks of this device's compute peaks in TFLOP/s, the denominators of compute-bound rooflines: kind 0 the
 * fp32 FMA rate of the SIMT lanes (register-only FFMA loop at full occupancy), kind 1 the tf32 rate of the tensor
 * cores (tcgen05.mma kind::tf32, M = 128, N = 256, operands in shared memory), kind 2 the fp32 rate with packed
 * two-wide FMAs (fma.rn.f32x2), kind 16 .. 256 (a multiple of 16) the
 * tensor-core rate with N = kind, which shows the instruction-rate limit of narrow tiles.  A few milliseconds each.  Diagnostics;
 * no counterpart in the reference. */
int grace_measure_peak(int kind, double *tflops);
/* _debug_track_alloc(on), _debug_peak_alloc(), _debug_live_alloc() (kk_module.cpp:221-224, kk_core.cpp:143-184): from
 * track_alloc(1) on every device allocation of the library is recorded by label; peak = high-water mark in bytes of
 * the allocations made since then (the reference's torch-sim adapter sizes its batches from it,
 * python/grace_runtime/torchsim.py:143-148); live = "label<TAB>bytes" lines, largest first. */
int grace_debug_track_alloc(int on);
uint64_t grace_debug_peak_alloc(void);
int grace_debug_live_alloc(char *buf, size_t len);
const char *grace_last_error(void);            /* what() of the exception the reference would have thrown */
/* kernels launched by this library since the process started (diagnostics; no counterpart in the reference) */
uint64_t grace_kernel_launches(void);
/* per-kernel device time: with on != 0 every launch is bracketed by CUDA events on the launch stream; the report is
 * one "name launches total_ms" line per kernel since the profile was switched on, copied into buf (diagnostics; the
 * reference labels its kernels for external profilers instead) */
int grace_profile_enable(int on);
int grace_profile_report(char *buf, size_t len);

/* Column sums of a row-major device matrix values[n][k] of doubles (per-atom energies, k = 1, or per-atom virial rows,
 * k = 6, to totals) into out[k] on the device, WITHOUT any device allocation.  No counterpart in the reference.
 * The per-block partial sums live in one statically allocated device array (65,792 bytes per device) instead of
 * allocator memory, for callers that cannot allocate when they need the sum: a host code that has given all free
 * device memory to its own pool, or a time-step loop that must not meet the device-wide synchronisation an
 * allocation can imply.  Limits: k <= 8, n <= 16,777,216 rows; larger sizes return GRACE_INVALID_ARGUMENT.
 * Deterministic (fixed summation tree).  Runs on the library's stream and returns after it has finished.  Every call
 * shares the array, so calls must not overlap in time on a device (the library's lock orders calls made through
 * this ABI).  The first call on a device also looks up the array's address: make it before any stream capture. */
int grace_sum_rows_static(const double *d_values, int64_t n, int k, double *d_out);

/* ---- Model (kk_api.h:51-64): a loaded GRACE-1L / GRACE-2L / GRACE-3L kokkos.npz ---- */
/* spline: intervals of the radial cubic Hermite tables (reference default 1024; >= 16), or 0: no tables, the exact
 * radial MLP per bond as in the reference's generic engine (tensor-core kernel; needs slots x outputs x 8 bytes of
 * device memory per layer and an 8 -> 64 -> 64 -> n radial MLP; GRACE-1L / 2L only).  GRACE-3L models evaluate on one
 * GPU through the System / Batch entry points below; the UQ flag, grace_system_set_owned / set_exchange and the engine
 * interface answer GRACE_UNSUPPORTED or GRACE_INVALID_ARGUMENT for them */
int grace_model_load(const char *path, int spline, grace_model **out);   /* Model(path, spline) */
int grace_model_layers(const grace_model *m);                            /* layers(): 1, 2 or 3 */
int grace_model_has_uq(const grace_model *m);                            /* has_uq(): the file carries a UQ head */
/* validate_uq() (kk_api.h:59): GRACE_OK, or GRACE_INVALID_ARGUMENT with the reason the head cannot be evaluated (none
 * in the file, a schema other than 6, a max_order 3 model, array sizes that do not match the model) */
int grace_model_validate_uq(const grace_model *m);
int grace_model_n_elements(const grace_model *m);                        /* len(element_names()) */
const char *grace_model_element_name(const grace_model *m, int i);       /* element_names()[i] */
int64_t grace_model_engine_setups(const grace_model *m);                 /* engine_setups() */
/* fp32 flops per atom of the dense network (FC layers, products, reduces; forward and reverse programs, each once)
 * of the engine's plan; 0 before the first System / Batch of the model.  Diagnostics for roofline figures; no
 * counterpart in the reference. */
double grace_model_dense_flops(const grace_model *m);
/* Per atom and evaluation on the per-operation path of the dense network (each program of each layer once):
 * out6 = {useful flops, algorithmic bytes} of the operations on the tensor cores, of the products, of the per-element
 * operations (bytes: every input row once per item or tensor, every output row once, twice when it accumulates).
 * Needs an engine (a System or Batch of the model).  Diagnostics for roofline figures. */
int grace_model_dense_stats(const grace_model *m, double *out6);
/* The exact radial MLP of layer 1 or 2 (no tables) for nb scaled distances x = r / r_cut in (0, 1): value R[nb][w] and
 * derivative dR/dx [nb][w] with w = grace_model_radial_mlp_width(), outputs ordered [l][channel]; device pointers, fp32.
 * Runs as tcgen05 tensor-core GEMMs with fused activations (shapes: up to 8 basis functions, two hidden layers of 64,
 * w a multiple of 32 up to 192; other shapes return GRACE_UNSUPPORTED).  Counterpart of compute_mlp_radial of the
 * reference's generic engine (libgrace/include/grace/kk/grace_1l_kk_impl.h:1592-1751). */
int grace_model_radial_mlp_device(grace_model *m, int layer, int64_t nb, const float *d_x, float *d_R, float *d_dR);
int grace_model_radial_mlp_width(const grace_model *m, int layer);
void grace_model_free(grace_model *m);

/* ---- System (kk_api.h:68-90): one structure, neighbour list with a Verlet skin kept on the device ---- */
/* spline: radial mode of this System, as the reference's System argument (kk_api.h:75; the reference ignores the
 * Model's value, python/kk/kk_core.cpp:321): > 0 cubic Hermite tables with that many intervals (>= 16, default 1024);
 * 0 the exact radial MLP per bond; < 0 the value the model was loaded with.  Systems and Batches of one model that ask
 * for the same spline share one device engine; grace_model_engine_setups() counts the engines built.
 * chunksize: atoms per engine pass (0: all atoms in one pass; < 0: chosen from the free device memory) */
int grace_system_create(const grace_model *m, const char *const *species, int n_species, double skin, int spline,
                        int chunksize, grace_system **out);              /* System(model, species, skin, spline, chunk) */
double grace_system_cutoff(const grace_system *s);                        /* cutoff() */
/* System::compute: host arrays in, host arrays out.  energy [1]; virial6 [6], forces [n][3] (skipped with
 * GRACE_FLAG_ENERGY_ONLY); energies [n] (with GRACE_FLAG_ENERGIES).  Null output pointers are skipped. */
int grace_system_compute(grace_system *s, int n, const int32_t *types, const double *pos, const double *cell,
                         const uint8_t *pbc, int flags, double *energy, double *virial6, double *forces,
                         double *energies);
/* the same with device pointers for types, positions and every output (cell and pbc stay on the host); the
 * single-structure counterpart of Batch::compute_device (kk_api.h:139-145) */
int grace_system_compute_device(grace_system *s, int n, const int32_t *d_types, const double *d_pos,
                                const double *cell, const uint8_t *pbc, int flags, double *d_energy,
                                double *d_virial6, double *d_forces, double *d_energies);
/* Result::gamma / sigma / cluster (kk_api.h:39) and DeviceOut::gamma / sigma / cluster (kk_api.h:100): where the
 * calls with GRACE_FLAG_UQ from now on write the extrapolation grade, the Mahalanobis distance and the nearest
 * mixture component of every atom, [n] doubles each in the caller's atom order; host pointers for
 * grace_system_compute, device pointers for grace_system_compute_device.  The flag without all three pointers, or on a
 * model whose head grace_model_validate_uq rejects, is GRACE_INVALID_ARGUMENT (kk_core.cpp:826-827, 1284-1286).  A UQ
 * call evaluates the dense network on the per-operation path whatever the structure's size. */
int grace_system_set_uq_outputs(grace_system *s, double *gamma, double *sigma, double *cluster);
/* Domain decomposition: from now on only the atoms with index < nlocal are owned by this System; the atoms behind
 * them are ghosts (copies of atoms another rank owns), which enter every neighbour sum but whose own energies are
 * left out of `energy`, `energies` (0 there) and the gradient, while forces and virial of everything the owned
 * energies depend on are returned, ghost rows included, for the caller to send back to the owners.  The ghosts
 * [nlocal, ninner) are those whose layer-1 outputs owned atoms read (GRACE-2L: ghosts within cutoff + skin of an owned
 * atom; ninner < 0: all ghosts); ghosts behind ninner only serve as neighbours, and nothing but the neighbour list is
 * computed for them.  nlocal < 0: all atoms are owned (default).  Counterpart of nlocal / ghost atoms in the reference's engine input
 * (libgrace/include/grace/kk/grace_2l_kk.h:87-107) and of inum / ilist in its CPU drivers
 * (libgrace/include/grace/system.h:113-121); the plug-in interface kk_api.h itself is single-GPU. */
int grace_system_set_owned(grace_system *s, int nlocal, int ninner);
/* Diagnostics: the device neighbour list of the last build (radius cutoff + skin) copied to the host in the caller's
 * atom order: per bond the atoms bi, bj and the integer cell shift bS [3] with bond vector x_j - x_i + S cell.  *count
 * receives the number of bonds; nothing is written when capacity is smaller.  For bond-for-bond comparison with a CPU
 * search as the reference's own test does (tests/kk/test_kk_neighbors.cpp:1-6). */
int grace_system_neighbor_list(grace_system *s, int64_t capacity, int32_t *bi, int32_t *bj, int32_t *bS, int64_t *count);
int64_t grace_system_rebuilds(const grace_system *s);                     /* rebuilds() */
int grace_system_chunksize(const grace_system *s);                        /* chunksize() */
int grace_system_release_buffers(grace_system *s);                        /* release_device_buffers() */
/* device milliseconds of the stages of the last compute (CUDA events): [0] neighbour list, [1] bond geometry,
 * [2] forward, [3] reverse, [4] total; diagnostics of this backend (the reference exposes Batch::host_seconds) */
int grace_system_stage_ms(const grace_system *s, double *ms5);
void grace_system_free(grace_system *s);

/* ---- multi-GPU: one process per GPU, NCCL between the processes ----
 * Extension (kk_api.h is one GPU per process, python/kk/kk_core.cpp:86-98): the reference's multi-GPU runs go through
 * LAMMPS' ghost atoms with forward / reverse communication around its engine interface
 * (libgrace/include/grace/system.h:53-64, libgrace/include/grace/kk/grace_2l_kk.h:136-153).  Here a host code splits the
 * structure into domains, gives every rank its owned atoms followed by a ghost halo of layers x (cutoff + skin), and
 * the library returns the ghost force rows to their owners and sums energy and virial inside the compute call, on its
 * own stream (ncclSend / ncclRecv pairs and one 7-value all-reduce; NCCL is loaded at run time from libnccl.so.2).
 * grace_comm_unique_id: rank 0 fills 128 bytes the caller passes to every rank (any transport);
 * grace_comm_init: every rank, after grace_initialize; collective.  One communicator per process. */
int grace_comm_unique_id(void *id128);
int grace_comm_init(const void *id128, int rank, int world);
int grace_comm_finalize(void);
int grace_comm_rank(void);                                                /* -1 without a communicator */
int grace_comm_size(void);                                                /* 0 without a communicator */
/* Exchange plan of a decomposed System of n atoms: atoms [0, nlocal) owned, [nlocal, ninner) ghosts whose layer-1
 * outputs owned atoms read, the rest neighbours only (as grace_system_set_owned).  send_index: indices (into the n atoms)
 * of the ghost atoms whose force rows leave, grouped by owner rank, send_counts[world] rows per rank; recv_index: for the
 * rows arriving from rank 0, 1, ... in that order (recv_counts[world]), the owned atom each is added to.  After it, every
 * compute of the system is collective: forces of owned atoms, energy and virial are the totals of the structure. */
int grace_system_set_exchange(grace_system *s, int n, int nlocal, int ninner, const int32_t *send_counts,
                              const int32_t *send_index, const int32_t *recv_counts, const int32_t *recv_index);

/* ---- Engine interface for hosts with their own neighbour list and ghost atoms ----
 * The interface the reference's LAMMPS glue drives (RunInput / RunOutput / Exchange,
 * libgrace/include/grace/kk/grace_2l_kk.h:87-119; CPU side libgrace/include/grace/system.h:53-64): nall atoms, the nlocal
 * local ones first, then ghosts; the padded neighbour table of the local atoms over all atoms; forces are ADDED to
 * d_f [nall][3] including the ghost rows (the caller returns those to their owners, LAMMPS: reverse_comm), per-atom
 * energies to d_eatom [nlocal] (null: not wanted); energy and virial6 of the local atoms are returned on the host.
 * GRACE-2L needs the message rows of the ghosts: after layer 1 `forward` must copy the rows of the owners into their
 * ghosts, before layer 1 is reversed `reverse` must add the rows of the ghosts into their owners (rows: device,
 * [nall][width] fp32, width = grace_engine_comm_width(); stream: the library's cudaStream_t, idle when the hook is
 * called).  Null hooks: no ghost is an image of a local atom.  All pointers of grace_run_input are device pointers. */
typedef struct grace_engine grace_engine;
typedef void (*grace_exchange_fn)(void *user, float *d_rows, int width, void *stream);
typedef struct {
  int nlocal, nall;
  const int32_t *d_type;         /* [nall] 1-based types into species */
  const double *d_x;             /* [nall][3] */
  const int32_t *d_numneigh;     /* [nlocal] */
  const int32_t *d_neighbors;    /* [nlocal][maxneigh] indices into the nall atoms */
  int maxneigh;
  int flags;                     /* GRACE_FLAG_ENERGY_ONLY */
  grace_exchange_fn forward, reverse;
  void *user;
} grace_run_input;
int grace_engine_create(const grace_model *m, const char *const *species, int n_species, int spline, int chunksize,
                        grace_engine **out);                              /* set_model + setup */
double grace_engine_cutoff(const grace_engine *e);
int grace_engine_comm_width(const grace_engine *e);                       /* comm_width() */
int grace_engine_run(grace_engine *e, const grace_run_input *in, double *energy, double *virial6, double *d_f,
                     double *d_eatom);                                    /* run(RunInput) -> RunOutput */
void grace_engine_free(grace_engine *e);

/* ---- Batch (kk_api.h:92-156): many structures per engine pass ---- */
int grace_batch_create(const grace_model *m, const char *const *species, int n_species, int spline, int chunksize,
                       grace_batch **out);                                /* Batch(model, species, spline, chunk) */
double grace_batch_cutoff(const grace_batch *b);
/* Batch::compute: natoms [nsys]; types [ntot]; pos [ntot][3]; cell [nsys][3][3]; pbc [nsys][3]; max_nall: atoms per
 * engine pass (whole structures per pass; <= 0: the reference default 2^21).  energy [nsys]; virial [nsys][6];
 * forces [ntot][3]; energies [ntot] */
int grace_batch_compute(grace_batch *b, int nsys, const int32_t *natoms, int64_t ntot, const int32_t *types,
                        const double *pos, const double *cell, const uint8_t *pbc, int flags, int64_t max_nall,
                        double *energy, double *virial, double *forces, double *energies);
/* Batch::compute_device: types, pos and the outputs are device pointers of the initialised GPU */
int grace_batch_compute_device(grace_batch *b, int nsys, const int32_t *natoms, int64_t ntot, const int32_t *d_types,
                               const double *d_pos, const double *cell, const uint8_t *pbc, int flags,
                               int64_t max_nall, double *d_energy, double *d_virial, double *d_forces,
                               double *d_energies);
/* as grace_system_set_uq_outputs, [ntot] doubles each (BatchResult / DeviceOut, kk_api.h:96,105) */
int grace_batch_set_uq_outputs(grace_batch *b, double *gamma, double *sigma, double *cluster);
int grace_batch_passes(const grace_batch *b);                             /* passes() */
double grace_batch_host_seconds(const grace_batch *b);                    /* host_seconds() */
int grace_batch_set_keep_buffers(grace_batch *b, int on);                 /* set_keep_buffers(on) */
int grace_batch_release_buffers(grace_batch *b);                          /* release_device_buffers() */
void grace_batch_free(grace_batch *b);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif
