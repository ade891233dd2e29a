// A kernel written outside the library with its device primitives: every rank fills
// a vector, all-reduces it with the device function tile_allreduce, passes a token
// to its right neighbour with tile_put + tile_signal / tile_wait, and meets the
// others in tile_barrier.  Compile and run it with examples/custom_kernel.py.
//
// One CTA acts as one rank.  Launched with one CTA per GPU, `w.rank` is the rank of
// that GPU; launched as ONE cooperative grid of world_size CTAs on a single GPU, CTA
// r plays rank r (args.v[4] = 1 selects that form), which is how the kernel can be
// tried without a second GPU: a cooperative grid is resident as a whole, so its CTAs
// may wait for one another.
//
// args: v[0] data   float[n] on the heap (symmetric)      v[1] n
//       v[2] sync   uint32[64] on the heap (symmetric, zero before the first call):
//                   [0, 32) collective counter block, [32] barrier counter, [33] token flag
//       v[3] epoch  1, 2, 3 ... per call                   v[4] 1 = CTA index is the rank
//       v[5] token  uint32[4] on the heap (symmetric)     v[6] status uint32[8] (local)
#include <tile_collectives.cuh>
#include <user_kernel.cuh>

using namespace tileccl;

__global__ void ring_allreduce_demo(SymmWindow w, UserArgs a) {
  __shared__ uint32_t abort_word;
  if (threadIdx.x == 0) abort_word = 0;
  __syncthreads();
  if (a.v[4] != 0) {
    // Emulated ranks: CTA r works in rank r's heap.  Symmetric arguments are addresses in
    // rank 0's heap; translate them to this rank's copy.
    w.rank = static_cast<int>(blockIdx.x);
  }
  auto mine = [&](int i) { return translate_ptr(w, reinterpret_cast<char*>(a.v[i]), 0, a.v[4] ? w.rank : 0); };
  float* data = reinterpret_cast<float*>(mine(0));
  const uint64_t n = a.v[1];
  uint32_t* sync = reinterpret_cast<uint32_t*>(mine(2));
  const uint32_t epoch = static_cast<uint32_t>(a.v[3]);
  uint32_t* token = reinterpret_cast<uint32_t*>(mine(5));
  uint32_t* status = reinterpret_cast<uint32_t*>(a.v[6]);

  WaitBudget wb;
  wb.start(1000000000ull, &abort_word);   // every wait gives up after one second

  // 1. rank r contributes (r + 1) * (i % 7 + 1) to element i
  for (uint64_t i = threadIdx.x; i < n; i += blockDim.x)
    data[i] = static_cast<float>(w.rank + 1) * static_cast<float>(i % 7 + 1);
  __syncthreads();

  // 2. all-reduce in place (announce -> wait -> pull, sum, push -> publish -> wait)
  TileCollSync cs{sync, epoch, status, -1};
  bool ok = tile_allreduce(w, data, n * sizeof(float), kTileF32, /*use_mc=*/false, cs, wb);

  // 3. token ring: put one word into the right neighbour's heap, raise its flag, wait for ours
  const int right = (w.rank + 1) % w.world_size;
  if (threadIdx.x == 0) {
    token[1] = 1000u * epoch + static_cast<uint32_t>(w.rank);          // what we send
    TileView src{reinterpret_cast<char*>(token + 1), 16, 1, 4};
    TileView dst{reinterpret_cast<char*>(token), 16, 1, 4};            // lands in token[0] there
    tile_put(w, src, dst, right, 0, 1);
    tile_signal(w, sync + 33, right);                                  // release: the put is visible first
    ok = tile_wait(sync + 33, wb) && ok;                               // consume our own flag
    // 4. everybody meets before anyone reuses the buffers
    ok = tile_barrier(w, sync + 32, epoch, wb) && ok;
    if (!ok) report_status(status, kStatusTimeoutSignal, 90, epoch, 0, w.rank, 0);
  }
}

TILECCL_USER_KERNEL_MAIN_COOPERATIVE(ring_allreduce_demo)
