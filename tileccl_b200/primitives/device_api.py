"""Names of the device-side tile primitives.

In the reference these are ``@triton.jit`` functions (tileccl/primitives/
memory.py, communication.py, compute.py; tileccl/sync/primitives.py).  Here the
primitives are CUDA ``__device__`` functions for sm_100a in ``csrc/device/*.cuh``
and are meant to be included by CUDA kernels.  This module keeps every name
importable from Python (``from tileccl.primitives import tile_put``) and says
where the implementation lives; calling one from the host raises.

To use them, write a ``.cu`` kernel that includes the headers and build / launch it
with :mod:`tileccl_b200.userkernel` (``examples/custom_kernel.cu`` shows one).  The
host-callable test harness for single primitives is
:mod:`tileccl_b200.primitives.harness`.
"""

from __future__ import annotations


class DevicePrimitive:
    """Documentation stub of a CUDA device function."""

    def __init__(self, name: str, header: str, signature: str, doc: str):
        self.__name__ = name
        self.name = name
        self.header = header
        self.signature = signature
        self.__doc__ = f"{doc}\n\nCUDA: ``{signature}`` in ``csrc/device/{header}``."

    def __call__(self, *args, **kwargs):
        raise RuntimeError(
            f"{self.name} is a CUDA device function (csrc/device/{self.header}); include the header "
            "in a kernel (tileccl_b200.userkernel compiles and launches one), or drive it from "
            "Python through tileccl_b200.primitives.harness")

    def __repr__(self) -> str:
        return f"<device primitive {self.name} ({self.header})>"


def _p(name, header, signature, doc):
    return DevicePrimitive(name, header, signature, doc)


# ---- memory ------------------------------------------------------------------
tile_load = _p("tile_load", "tile_mem.cuh",
               "int tile_load(const TileView& src, uint4 (&frag)[N], int tid, int nthreads)",
               "Cooperative load of a tile into per-thread 16-byte fragments.")
tile_store = _p("tile_store", "tile_mem.cuh",
                "void tile_store(const TileView& dst, const uint4 (&frag)[N], int tid, int nthreads)",
                "Cooperative store of per-thread fragments into a tile.")
tile_copy = _p("tile_copy", "tile_mem.cuh",
               "void tile_copy(const TileView& dst, const TileView& src, int tid, int nthreads)",
               "Cooperative tile-to-tile copy with predicated tails.")
make_block_offsets = _p("make_block_offsets", "tile_mem.cuh",
                        "TileView make_tile_view(void* base, int64_t ld, int elem_bytes, int row0, "
                        "int col0, int bm, int bn, int rows, int cols)",
                        "Describe a BMxBN tile of a row-major matrix (clipped at the edges).")
# ---- communication -----------------------------------------------------------
translate_ptr = _p("translate_ptr", "symm_ptr.cuh",
                   "T* translate_ptr(const SymmWindow& w, T* p, int from_rank, int to_rank)",
                   "Same heap object on another rank: p + (to - from) * stride.")
remote_load = _p("remote_load", "symm_ptr.cuh", "uint4 ld_remote_v4(const void* p)",
                 "16-byte load that bypasses L1 (peer-written data is never stale).")
remote_store = _p("remote_store", "symm_ptr.cuh", "void st_remote_v4(void* p, const uint4& v)",
                  "16-byte store to a (possibly remote) address.")
tile_remote_load = _p("tile_remote_load", "tile_comm.cuh",
                      "int tile_remote_load(const SymmWindow&, const TileView& sym_src, int from_rank, "
                      "uint4 (&frag)[N], int tid, int nthreads)",
                      "Peer memory -> registers.")
tile_remote_store = _p("tile_remote_store", "tile_comm.cuh",
                       "void tile_remote_store(const SymmWindow&, const TileView& sym_dst, int to_rank, "
                       "const uint4 (&frag)[N], int tid, int nthreads)",
                       "Registers -> peer memory.")
tile_put = _p("tile_put", "tile_comm.cuh",
              "void tile_put(const SymmWindow&, const TileView& src, const TileView& sym_dst, "
              "int to_rank, int tid, int nthreads)", "Local memory -> peer memory.")
tile_get = _p("tile_get", "tile_comm.cuh",
              "void tile_get(const SymmWindow&, const TileView& sym_src, const TileView& dst, "
              "int from_rank, int tid, int nthreads)", "Peer memory -> local memory.")
tile_put_mc = _p("tile_put_mc", "tile_comm.cuh",
                 "void tile_put_mc(const SymmWindow&, const TileView& src, const TileView& sym_dst, "
                 "int tid, int nthreads)", "One multimem.st per 16 bytes lands the tile on every rank.")
tile_get_reduce = _p("tile_get_reduce", "tile_comm.cuh",
                     "void tile_get_reduce(const SymmWindow&, const TileView& sym_src, "
                     "const TileView& dst, int kind, int tid, int nthreads)",
                     "multimem.ld_reduce: sum of the tile over all ranks (fp32 accumulation).")
# ---- compute -----------------------------------------------------------------
tile_dot = _p("tile_dot", "../kernels/gemm_sm100.cu",
              "tcgen05.mma main loop of fused_gemm_sm100_kernel",
              "Matrix product of tiles: issued by the tcgen05 main loop, not a free function.")
tile_reduce = _p("tile_reduce", "tile_compute.cuh", "float tile_reduce(const float (&v)[N], int mode)",
                 "Sum / max / min of a warp's register tile.")
tile_reduce_max = tile_reduce
tile_reduce_min = tile_reduce
tile_elementwise = _p("tile_elementwise", "tile_compute.cuh",
                      "void tile_elementwise(int op, float (&v)[N])",
                      "exp / log / abs / neg / sqrt / relu / sigmoid / silu on a register tile.")
tile_cast = _p("tile_cast", "tile_compute.cuh", "uint4 tile_cast_f32x8(bool is_bf16, const float* v)",
               "fp32 -> packed fp16 / bf16.")
tile_zeros = _p("tile_zeros", "tile_compute.cuh", "void tile_zeros(float (&v)[N])", "Zero a register tile.")
tile_full = _p("tile_full", "tile_compute.cuh", "void tile_full(float (&v)[N], float x)",
               "Fill a register tile.")
# ---- synchronisation ---------------------------------------------------------
_SYNC = "tile_sync.cuh"
tile_atomic_add = _p("tile_atomic_add", _SYNC, "uint32_t tile_atomic_add(w, target, value, to_rank)", "Remote atomic add.")
tile_atomic_cas = _p("tile_atomic_cas", _SYNC, "uint32_t tile_atomic_cas(w, target, compare, value, to_rank)", "Remote compare-and-swap.")
tile_atomic_xchg = _p("tile_atomic_xchg", _SYNC, "uint32_t tile_atomic_xchg(w, target, value, to_rank)", "Remote exchange.")
tile_atomic_min = _p("tile_atomic_min", _SYNC, "uint32_t tile_atomic_min(w, target, value, to_rank)", "Remote atomic min.")
tile_atomic_max = _p("tile_atomic_max", _SYNC, "uint32_t tile_atomic_max(w, target, value, to_rank)", "Remote atomic max.")
tile_atomic_and = _p("tile_atomic_and", _SYNC, "uint32_t tile_atomic_and(w, target, value, to_rank)", "Remote atomic and.")
tile_atomic_or = _p("tile_atomic_or", _SYNC, "uint32_t tile_atomic_or(w, target, value, to_rank)", "Remote atomic or.")
tile_atomic_xor = _p("tile_atomic_xor", _SYNC, "uint32_t tile_atomic_xor(w, target, value, to_rank)", "Remote atomic xor.")
tile_signal = _p("tile_signal", _SYNC, "void tile_signal(w, flag, to_rank)",
                 "Release-store 1 into a peer's flag.")
tile_wait = _p("tile_wait", _SYNC, "bool tile_wait(flag, const WaitBudget&)",
               "Bounded acquire-wait that consumes the flag (1 -> 0).")
tile_try_wait = _p("tile_try_wait", _SYNC, "bool tile_try_wait(flag, int max_spins)",
                   "Poll-count bounded consuming wait.")
tile_poll = _p("tile_poll", _SYNC, "bool tile_poll(flag, const WaitBudget&)", "Bounded non-consuming wait.")
tile_try_poll = _p("tile_try_poll", _SYNC, "bool tile_try_poll(flag, int max_spins)",
                   "Poll-count bounded non-consuming wait.")
tile_signal_add = _p("tile_signal_add", _SYNC, "void tile_signal_add(w, counter, amount, to_rank)",
                     "Release-add to a peer's counter.")
tile_wait_ge = _p("tile_wait_ge", _SYNC, "bool tile_wait_ge(counter, target, const WaitBudget&, observed)",
                  "Bounded wait until a local counter reaches a target (wrap-safe).")
tile_acquire_credit = _p("tile_acquire_credit", _SYNC, "bool tile_acquire_credit(credits, const WaitBudget&)",
                         "Take one credit from a local pool.")
tile_release_credit = _p("tile_release_credit", _SYNC, "void tile_release_credit(w, credits, to_rank)",
                         "Give one credit back to a peer's pool.")
tile_barrier = _p("tile_barrier", _SYNC, "bool tile_barrier(w, counter, epoch, const WaitBudget&)",
                  "All-ranks barrier on a counter that only grows.")
# ---- collectives as device building blocks -------------------------------------
_COLL = "tile_collectives.cuh"
tile_allreduce = _p("tile_allreduce", _COLL,
                    "bool tile_allreduce(w, sym_buf, bytes, dtype, use_mc, const TileCollSync&, const WaitBudget&)",
                    "In-place sum over all ranks: announce, wait, pull-sum-push own share, publish, wait "
                    "(data phase alone: tile_allreduce_chunk).")
tile_allgather = _p("tile_allgather", _COLL,
                    "void tile_allgather(w, src, sym_dst, bytes, elem_size, use_mc, TileCoop) / "
                    "bool tile_allgather(..., const TileCollSync&, const WaitBudget&)",
                    "Own chunk into slot `rank` of every rank's output (multimem.st with NVLS).")
tile_scatter = _p("tile_scatter", _COLL,
                  "void tile_scatter(w, src, sym_dst, bytes, root, elem_size, TileCoop) / "
                  "bool tile_scatter(..., const TileCollSync&, const WaitBudget&)",
                  "Root pushes chunk r to rank r.")
tile_reduce_scatter = _p("tile_reduce_scatter", _COLL,
                         "void tile_reduce_scatter(w, sym_src, dst, bytes, dtype, use_mc, TileCoop) / "
                         "bool tile_reduce_scatter(..., const TileCollSync&, const WaitBudget&)",
                         "Sum of chunk `rank` over all ranks into a local buffer (multimem.ld_reduce with NVLS).")
tile_broadcast = _p("tile_broadcast", _COLL,
                    "void tile_broadcast(w, sym_buf, bytes, root, elem_size, use_mc, TileCoop) / "
                    "bool tile_broadcast(..., const TileCollSync&, const WaitBudget&)",
                    "Root's buffer into the same place of every other rank's heap.")

MEMORY = ["tile_load", "tile_store", "tile_copy", "make_block_offsets"]
COMMUNICATION = ["translate_ptr", "remote_load", "remote_store", "tile_remote_load",
                 "tile_remote_store", "tile_put", "tile_get", "tile_put_mc", "tile_get_reduce"]
COMPUTE = ["tile_dot", "tile_reduce", "tile_reduce_max", "tile_reduce_min", "tile_elementwise",
           "tile_cast", "tile_zeros", "tile_full"]
SYNC = ["tile_atomic_add", "tile_atomic_cas", "tile_atomic_xchg", "tile_atomic_min", "tile_atomic_max",
        "tile_atomic_and", "tile_atomic_or", "tile_atomic_xor", "tile_signal", "tile_wait",
        "tile_try_wait", "tile_poll", "tile_try_poll", "tile_signal_add", "tile_wait_ge",
        "tile_acquire_credit", "tile_release_credit", "tile_barrier"]
COLLECTIVE_DEVICE = ["tile_allreduce", "tile_allgather", "tile_scatter", "tile_reduce_scatter",
                     "tile_broadcast"]
