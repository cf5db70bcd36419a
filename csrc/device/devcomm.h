// Structures shared by host and device code of the cuda transport.
//
// Every communicator owns a *control block* in symmetric memory (same layout on every rank, every rank
// maps every peer's copy).  It holds the flags through which the kernels of different GPUs synchronise,
// the one-shot exchange slots and the Send/Recv FIFOs.  All flags are monotonically increasing 64-bit
// counters, never reset, so back-to-back collectives cannot confuse one call's signal with the next.
#pragma once

#include <stdint.h>

#define MCCL_MAX_RANKS 16      // ranks of one NVSwitch domain a kernel can address
#define MCCL_P2P_DEPTH 4       // chunks of a Send/Recv channel's ring in the receiver's memory
#define MCCL_P2P_CHANNELS 32   // most CTAs that share one Send/Recv message (each with its own part of the FIFO slot)
#define MCCL_MAX_CTAS 160      // upper bound on CTAs ("channels") of one collective kernel
#define MCCL_COLL_THREADS 512
#define MCCL_ONESHOT_MAX_CTAS 8   // the one-shot kernel never runs more CTAs: its call counters are kept equal over this many

#ifdef __CUDACC__
#define MCCL_HD __host__ __device__
#else
#define MCCL_HD
#endif

namespace mccl {

// Device status word (pinned host memory, one per communicator).  A wait that runs out of time records
// where it gave up and the kernel returns normally; nothing traps.
struct DevStatus {
  volatile uint32_t code;     // 0 = fine, 1 = timeout in a barrier, 2 = timeout in a step wait, 3 = aborted by host,
                              // 4 = the ranks disagree on the buffers of a call (MCCL_CHECK_SYMMETRY)
  volatile uint32_t peer;     // rank that did not answer
  volatile uint32_t cta;
  volatile uint32_t step;
  volatile uint32_t abort;    // host sets it to make every wait give up at once
  uint32_t pad[3];
};

struct CtrlFlags {
  // bar[cta][src]: written by rank `src`'s CTA `cta`: "I have reached barrier number N".
  uint64_t bar[MCCL_MAX_CTAS][MCCL_MAX_RANKS];
  // sig[cta][src]: step signals of the ring / tree kernels, written by rank `src`.
  uint64_t sig[MCCL_MAX_CTAS][MCCL_MAX_RANKS];
  // epoch[cta]: barriers this rank's CTA has passed so far (local bookkeeping, read at kernel entry).
  uint64_t epoch[MCCL_MAX_CTAS];
  // one-shot: ready[cta][src] = number of one-shot calls whose data from `src` has fully arrived.
  uint64_t oneShotReady[MCCL_MAX_CTAS][MCCL_MAX_RANKS];
  // oneShotCalls[cta]: one-shot calls made so far.  Every launch leaves the first MCCL_ONESHOT_MAX_CTAS entries
  // equal, whatever its grid, so the slot half a call uses (its parity) is the same for every CTA.
  uint64_t oneShotCalls[MCCL_MAX_CTAS];
  // Send/Recv FIFOs, one per (peer, channel): head[src][ch] = chunks rank `src` has written into channel `ch` of
  // my slot; tail[dst][ch] = chunks rank `dst` has drained from its slot for me.  sent/recvd are this rank's own
  // running totals.
  uint64_t p2pHead[MCCL_MAX_RANKS][MCCL_P2P_CHANNELS];
  uint64_t p2pTail[MCCL_MAX_RANKS][MCCL_P2P_CHANNELS];
  uint64_t p2pSent[MCCL_MAX_RANKS][MCCL_P2P_CHANNELS];
  uint64_t p2pRecvd[MCCL_MAX_RANKS][MCCL_P2P_CHANNELS];
  // note[cta]: a word the root of a rooted collective publishes before the entry barrier of a call and its
  // peers read after it (which form of the algorithm the root can take part in).
  uint64_t note[MCCL_MAX_CTAS];
  // symSig[src]: what rank `src` passed to the call being checked (MCCL_CHECK_SYMMETRY): which symmetric
  // allocation and offset its send and receive buffers are, the collective and the count.
  uint64_t symSig[MCCL_MAX_RANKS][4];
  uint64_t canary;            // 0x6d63636c63616e61, checked by tests after every run
};

constexpr uint64_t kCanary = 0x6d63636c63616e61ull;

// Layout of the control segment: flags, then the one-shot slots, then the Send/Recv slots.
struct CtrlLayout {
  uint64_t flagsOff;
  uint64_t oneShotOff;      // 2 buffers x n ranks x oneShotSlotBytes
  uint64_t oneShotSlotBytes;
  uint64_t p2pOff;          // n ranks x p2pSlotBytes (channels x MCCL_P2P_DEPTH chunks each)
  uint64_t p2pSlotBytes;
  uint64_t stageOff;        // staging area for buffers that are not symmetric
  uint64_t stageBytes;
  uint64_t totalBytes;
};

struct DevPeers {
  int rank, n;
  char* ctrl[MCCL_MAX_RANKS];     // every rank's control segment as mapped here (ctrl[rank] = local)
  char* ctrlMc;                   // multicast alias of the control segment, or null
  CtrlLayout layout;
  DevStatus* status;              // device alias of the pinned status word
  uint64_t timeoutNs;
};

struct CopyJob {
  const char* src;
  char* dst;
  uint64_t bytes;
};

// Arguments of the pull kernel (two-shot all-reduce and every "direct" collective).
struct PullArgs {
  DevPeers peers;
  int nCtas;
  int op;                      // mcclRedOp_t
  // phase A: fold `nSrcA` sources over [aBytes) into dstA (and dstA2 if set)
  int nSrcA;
  const char* srcA[MCCL_MAX_RANKS];
  char* dstA;
  char* dstA2;
  uint64_t aBytes;
  // phase B: plain copies, each sliced over the CTAs
  int nJobs;
  CopyJob jobs[MCCL_MAX_RANKS + 1];
  int divisor;                 // avg: number of ranks, else 1
  int midBarrier;              // barrier between the phases (same value on every rank of a call)
};

struct OneShotArgs {
  DevPeers peers;
  int nCtas;
  int op;
  const char* send;
  char* recv;
  uint64_t bytes;
  int divisor;
};

struct NvlsArgs {
  DevPeers peers;
  int nCtas;
  int op;
  int loadReduce;              // 1: read through multimem.ld_reduce from mcSrc; 0: read local src
  int mcStore;                 // 1: write through multimem.st to mcDst; 0: write local dst
  int active;                  // 0: this rank only takes part in the barriers
  const char* src;             // local source (loadReduce == 0)
  const char* mcSrc;
  char* dst;
  char* mcDst;
  uint64_t bytes;
  int divisor;
};

// Rooted NVLS collectives with the root's work spread over all ranks: every rank handles one shard.
//   broadcast: rank r loads shard r of the root's buffer (a peer load; the root reads its own memory) and
//              replicates it into every rank's copy with multimem.st;
//   reduce:    rank r lets the switch add shard r over all ranks (multimem.ld_reduce) and stores the sum
//              into the root's buffer (a peer store; the root writes its own memory).
// Only the root knows where its destination of a reduce lies.  It publishes `note` (destination minus its
// source, in bytes, when both lie in one symmetric allocation; kNoteAlone otherwise) and the peers add it
// to their mapping of the root's source; with kNoteAlone the root reduces the whole message by itself.
constexpr uint64_t kNoteAlone = 0x7fffffffffffffffull;
struct NvlsRootedArgs {
  DevPeers peers;
  int nCtas;
  int op;
  int root;
  int reducing;                // 1: reduce, 0: broadcast
  const char* rootBuf;         // the root's buffer as mapped here: source of a broadcast, the root's SOURCE of a reduce
  char* local;                 // root of a reduce: its destination
  const char* mcSrc;           // reduce: multicast alias of the source
  char* mcDst;                 // broadcast: multicast alias of the destination
  uint64_t bytes;              // whole message, a multiple of 16
  uint64_t note;               // reduce, root only
  int divisor;
};

struct RingArgs {
  DevPeers peers;
  int nCtas;
  int op;
  int prev, next;
  char* buf[MCCL_MAX_RANKS];   // every rank's work buffer (peer-visible), in place
  uint64_t bytes;
  int divisor;
  int phases;                  // bit 0: reduce-scatter steps, bit 1: all-gather steps (0 = both = all-reduce)
  int shift;                   // ring chunk c stands for the ((c - shift) mod n)-th part of the buffer; with
                               // shift 1 a rank ends the reduce phase owning (and starts the gather phase
                               // holding) its own part, which is what reduce-scatter / all-gather need
};

struct TreeArgs {
  DevPeers peers;
  int nCtas;
  int op;
  int up[2];
  int down[2][2];
  char* buf[MCCL_MAX_RANKS];
  uint64_t bytes;
  int divisor;
  int phases;                  // bit 0: up (fold towards the tree roots), bit 1: down (copy from the roots); 0 = both
};

// A group of all-reduce calls issued as ONE kernel: the CTAs walk the jobs between one entry and one exit barrier
// (plus one in the middle when any job takes the two-shot form), instead of one launch and two or three barriers
// per call.
struct GroupJob {
  const char* in[MCCL_MAX_RANKS];   // every rank's input as mapped here (two-shot)
  char* red[MCCL_MAX_RANKS];        // every rank's result as mapped here (two-shot)
  char* out;                        // this rank's result
  const char* mcIn;                 // multicast aliases (NVLS form), else null
  char* mcOut;
  uint64_t bytes;                   // a multiple of 16, at least 16 per rank
  int dt, op, divisor, nvls;
};
#define MCCL_MAX_GROUP_JOBS 12
struct GroupArgs {
  DevPeers peers;
  int nCtas;
  int nJobs;
  int anyTwoShot;
  GroupJob jobs[MCCL_MAX_GROUP_JOBS];
};

struct P2pDesc {
  int isSend;
  int peer;
  char* buf;
  uint64_t bytes;
};
#define MCCL_MAX_P2P_OPS 96
struct P2pArgs {
  DevPeers peers;
  int nOps;
  const P2pDesc* more;             // batches longer than MCCL_MAX_P2P_OPS: all descriptors, in device memory
  P2pDesc ops[MCCL_MAX_P2P_OPS];
};

// Send/Recv channels per flow for a communicator of n ranks: every CTA of a batch (2 (n - 1) flows at most) must fit
// the GPU at the same time, because a sender's CTAs wait for the peer's receiving CTAs and the other way round.
// 4 x 32, 6 x 20, 14 x 8 and 30 x 4 CTAs all fit 148 SMs at one CTA per SM.
MCCL_HD inline int p2pChannels(int n) { return n <= 3 ? 32 : n == 4 ? 20 : n <= 8 ? 8 : 4; }

// How one Send/Recv message of `bytes` bytes is cut: `channels` contiguous parts of `per` bytes (the last one takes
// what is left), each moved in chunks of `chunk` bytes through its channel's ring of MCCL_P2P_DEPTH chunks.  A pure
// function of the message size, the slot size and the communicator's size, so sender and receiver agree without
// talking; at least 64 KB per channel.
struct P2pSplit { int channels; uint64_t per; uint64_t half; };      // half: bytes of one chunk of the ring

MCCL_HD inline P2pSplit p2pSplit(uint64_t bytes, uint64_t slotBytes, int n) {
  P2pSplit sp;
  int maxCh = p2pChannels(n);
  sp.half = slotBytes / (MCCL_P2P_DEPTH * (uint64_t)maxCh) / 16 * 16;
  if (sp.half < 4096) { sp.half = slotBytes / MCCL_P2P_DEPTH / 16 * 16; maxCh = 1; }      // a slot too small to share
  const uint64_t want = (bytes + (64u << 10) - 1) / (64u << 10);
  sp.channels = (int)(want < (uint64_t)maxCh ? (want > 0 ? want : 1) : (uint64_t)maxCh);
  sp.per = ((bytes + sp.channels - 1) / sp.channels + 255) / 256 * 256;
  return sp;
}

// Shard r of a message of `bytes` bytes cut into n shards on 16-byte boundaries; the last shard takes the tail.
MCCL_HD inline uint64_t shardOff(uint64_t bytes, int n, int r) { return (uint64_t)(((unsigned __int128)(bytes / 16) * (unsigned)r) / (unsigned)n) * 16; }
MCCL_HD inline uint64_t shardEnd(uint64_t bytes, int n, int r) { return r == n - 1 ? bytes : shardOff(bytes, n, r + 1); }

}  // namespace mccl
