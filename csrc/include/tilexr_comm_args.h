// Device-visible communicator state ("CommArgs") and the geometry of a peer window.
//
// Every rank owns one window in its GPU's memory; every other rank of the communicator maps
// it (CUDA IPC between processes, plain peer access between threads of one process).  A
// kernel receives a pointer to its rank's CommArgs and reaches a peer through
// `peerMems[peer]`.  The same structure exists in the reference (src/include/comm_args.h:122-147);
// the layout here is sized for NVSwitch domains and adds the bounded-wait bookkeeping the
// reference lacks.
//
// Window layout (identical offsets on every rank):
//
//   [0, 1 MiB)            control block: abort word, grid barriers, done-epoch table,
//                         signal words (the "credit plane"), operator scratch
//   [1 MiB, 5 MiB)        flag area: 64-bit flags `(epoch << 32) | value`, never reset
//   [5 MiB, 7 MiB)        low-latency plane: two halves of 16-byte units {12 payload bytes, epoch}; nothing else is
//                         ever stored there, so a unit that carries the current epoch is this launch's data
//   [7 MiB, 7 MiB + D)    data half 0   \  launch with epoch m uses half (m & 1); the
//   [.., 7 MiB + 2D)      data half 1   /  done-epoch table guards reuse at m + 2
#ifndef TILEXR_COMM_ARGS_H
#define TILEXR_COMM_ARGS_H

#include <stdint.h>

#define TILEXR_MAX_RANK_SIZE 128
#define TILEXR_DFX_COUNT 50
#define TILEXR_PING_PONG_SIZE 2
#define TILEXR_COMM_BUFFER_SIZE_MB 1024          /* default 2*D */
#define TILEXR_MEMORY_DOMAIN_BUFFER_SIZE_MB 8    /* isolated small domain (reference: MemoryDomain) */
/* the same two sizes and the flag area under the reference's names (src/include/tilexr_types.h:25-31) */
#define TILEXR_COMM_BUFFER_SIZE TILEXR_COMM_BUFFER_SIZE_MB
#define TILEXR_MEMORY_DOMAIN_BUFFER_SIZE TILEXR_MEMORY_DOMAIN_BUFFER_SIZE_MB
#define TILEXR_INVALID_VALUE (-1LL)
#define TILEXR_MAX_REGISTERED_REGIONS 64

#define TILEXR_WIN_CTRL_OFFSET   0LL
#define TILEXR_WIN_CTRL_BYTES    (1LL << 20)
#define TILEXR_WIN_FLAG_OFFSET   (1LL << 20)
#define TILEXR_WIN_FLAG_BYTES    (4LL << 20)
#define TILEXR_FLAG_BUFF_BYTES TILEXR_WIN_FLAG_BYTES   /* the reference's name for the flag area */
#define TILEXR_WIN_LL_OFFSET     (5LL << 20)
#define TILEXR_WIN_LL_HALF_BYTES (1LL << 20)
#define TILEXR_WIN_DATA_OFFSET   (7LL << 20)
#define TILEXR_TILE_BYTES        (256LL << 10)   // pipelining granule of the tiled collectives

// Control block, in units of 64-bit words from the window base.
#define TILEXR_CTRL_ABORT_WORD        0          // epoch of a launch that gave up; peers write it
#define TILEXR_CTRL_GRIDBAR_WORD      8          // 16 x {uint32 count, uint32 generation}
#define TILEXR_CTRL_GRIDBAR_COUNT     16
#define TILEXR_CTRL_EPOCH_WORD        32         // epoch of the rank's last finished launch (GPU communicators)
#define TILEXR_CTRL_DONE_WORD         64         // doneEpoch[src], written by src at kernel end
#define TILEXR_CTRL_SCRATCH_WORD      1024       // operator scratch (counts, cursors), 56 KiB
#define TILEXR_CTRL_SCRATCH_WORDS     7168
#define TILEXR_CTRL_SIGNAL_OFFSET     (512LL << 10)   // signal plane, bytes from window base
#define TILEXR_CTRL_SIGNAL_BYTES      (512LL << 10)
#define TILEXR_SIGNAL_STRIDE          64              // one signal word per 64-byte line

// Flag area, in flag slots (8 bytes each) from TILEXR_WIN_FLAG_OFFSET.
#define TILEXR_FLAGS_PER_PAIR         1024       // ring slots per (source, destination) pair
#define TILEXR_FLAG_DATA_BASE         0          // "tile produced" flags  [src][slot]
#define TILEXR_FLAG_ACK_BASE          (TILEXR_MAX_RANK_SIZE * TILEXR_FLAGS_PER_PAIR)      // "tile consumed"
#define TILEXR_FLAG_OP_BASE           (2 * TILEXR_MAX_RANK_SIZE * TILEXR_FLAGS_PER_PAIR)  // operator specific
#define TILEXR_FLAG_OP_SLOTS          (TILEXR_MAX_RANK_SIZE * TILEXR_FLAGS_PER_PAIR)
// Slots indexed by the RECEIVER's own numbering (token*topK + k of a combine), written by whichever rank
// holds the row.  They get a plane of their own: in the planes above a slot belongs to one source, so a rank
// that has moved on to its next launch can only overwrite flags it wrote itself; a receiver-indexed slot in
// one of those planes could be hit by another rank's next launch before its real writer arrived.
#define TILEXR_FLAG_SLOT_BASE         (3 * TILEXR_MAX_RANK_SIZE * TILEXR_FLAGS_PER_PAIR)
#define TILEXR_FLAG_SLOT_SLOTS        (TILEXR_MAX_RANK_SIZE * TILEXR_FLAGS_PER_PAIR)

#ifdef __cplusplus
namespace TileXR {
#endif

// Capability bits in CommArgs::extraFlag.  On B200 every peer is one NVSwitch hop away, so
// there are no topology variants; the bits describe which mechanisms are usable.
enum TileXRExtraFlag {
    TILEXR_FLAG_P2P = 1u << 0,            // all peers are load/store reachable
    TILEXR_FLAG_NVLS = 1u << 1,           // an NVLink multicast alias of the window exists
    TILEXR_FLAG_DETERMINISTIC = 1u << 3,  // fixed-order reductions only (env LCCL_DETERMINISTIC)
    TILEXR_FLAG_SAME_PROCESS = 1u << 4,   // thread mode: peers are threads of this process
    TILEXR_FLAG_EMULATED = 1u << 5,       // several ranks share one GPU (test worlds)
    TILEXR_FLAG_TOPO_NVLINK = 1u << 6,    // every peer link is NVLink (native peer atomics)
    TILEXR_FLAG_TOPO_PCIE = 1u << 9,      // at least one peer is reached over PCIe peer-to-peer
    TILEXR_FLAG_RMA = 1u << 10,           // registered-memory put/get/signal available (UDMA analogue)
    TILEXR_FLAG_LOCAL_COPY = 1u << 11,    // device-initiated bulk local copy available (SDMA analogue)
    TILEXR_FLAG_MEMORY_ONLY = 1u << 18,   // memory domain: no signal plane users, no registry
    TILEXR_FLAG_HOST_MEMORY = 1u << 19,   // windows live in host shared memory (CPU plumbing mode)
};

// One registered region: a peer-visible allocation that every rank registered collectively.
struct TileXRRegion {
    uint64_t bytes;
    uint8_t *localBase;
    uint8_t **peerBase;    // device array [rankSize]: the region of rank r mapped here
    uint8_t *mcBase;       // the region through the NVLink multicast object (all ranks' copies at once), or null
};

#define TILEXR_REGISTRY_MAGIC 0x52525854u   // "TXRR"

struct TileXRRegistry {
    uint32_t magic;
    uint32_t version;
    uint32_t rankSize;
    uint32_t regionCount;
    struct TileXRRegion regions[TILEXR_MAX_REGISTERED_REGIONS];
};

struct CommArgs {
    int32_t rank;
    int32_t localRank;
    int32_t rankSize;
    int32_t localRankSize;       // ranks reachable by load/store (the NVSwitch domain)
    uint32_t extraFlag;
    int32_t commDomain;
    uint64_t peerMemBytes;       // bytes of one window
    uint64_t dataHalfBytes;      // D: bytes of one ping-pong data half
    uint64_t waitTimeoutNs;      // budget of every device-side wait
    uint64_t registrationGeneration;
    uint8_t *peerMems[TILEXR_MAX_RANK_SIZE];     // window of rank r, mapped in this rank's address space
    uint8_t *signalMems[TILEXR_MAX_RANK_SIZE];   // signal plane of rank r (inside its window)
    uint8_t *multicastMem;       // NVLS alias of the window, or null
    struct TileXRRegistry *registryPtr;          // device copy of the registry, or null
    void *localCopyWorkspace;    // bounce buffer for device-initiated local copies, or null
    void *dumpAddr;
    int64_t dfx[TILEXR_DFX_COUNT];               // written by kernels, printed by TileXRPrintDFX2Log
};

// dfx[] slots.
enum TileXRDfxSlot {
    TILEXR_DFX_MAGIC = 0,
    TILEXR_DFX_OP = 1,
    TILEXR_DFX_COUNT_ARG = 2,
    TILEXR_DFX_RUN_STATUS = 3,     // 0xbeef while running, 0xd0e when finished, 0xdead on failure
    TILEXR_DFX_FAIL_CODE = 4,      // TileXRDeviceStatus
    TILEXR_DFX_FAIL_PEER = 5,
    TILEXR_DFX_FAIL_SLOT = 6,
    TILEXR_DFX_FAIL_EXPECTED = 7,
    TILEXR_DFX_FAIL_OBSERVED = 8,
    TILEXR_DFX_FAIL_BLOCK = 9,
    TILEXR_DFX_LAUNCHES = 10,
    // Phase times of the last topology-aware planner launch on this rank, ns: mail exchange, validation and table set-up,
    // balancing, per-route destinations, consensus and stage tables.
    TILEXR_DFX_PLAN_PHASE_NS = 16,     // five entries
};

#define TILEXR_RUN_STARTED  0xbeefLL
#define TILEXR_RUN_FINISHED 0x0d0eLL
#define TILEXR_RUN_FAILED   0xdeadLL

// Status a device-side wait leaves behind.  Zero means success.
enum TileXRDeviceStatus {
    TILEXR_DEV_OK = 0,
    TILEXR_DEV_WAIT_TIMEOUT = 1,      // the flag never reached the expected value
    TILEXR_DEV_ABORTED = 2,           // another block or rank raised the abort word
    TILEXR_DEV_BAD_RANGE = 3,         // a put/get touched memory outside its registered region
    TILEXR_DEV_BAD_ARGUMENT = 4,
    TILEXR_DEV_GRID_BARRIER_TIMEOUT = 5,
    TILEXR_DEV_REUSE_GUARD_TIMEOUT = 6,   // a peer never finished the launch two epochs ago
    TILEXR_DEV_MBARRIER_TIMEOUT = 7,
};

#ifdef __cplusplus
} // namespace TileXR
#endif

#endif // TILEXR_COMM_ARGS_H
