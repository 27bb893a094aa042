// Protocol checker: runs the flag protocols of this runtime on the CPU, rank by rank, records
// every copy / read / flag store / flag wait as an event, and analyses the event log for
// ordering bugs.  No GPU is involved; several "servers" can be modelled in one process.
//
// It is the counterpart of the reference's tilexr_checker (tools/checker/README.md,
// include/tilexr/checker/{event,world,executor,diagnostics}.h): same event model, same
// finding classes, same idea of fault-injection switches that flip one protocol step so that
// every rule has a positive test.  The executors model THIS runtime's protocols (push tiles,
// epoch flags, count-first EP placement), not the reference's kernels.
#ifndef TILEXR_CHECKER_H
#define TILEXR_CHECKER_H

#include <cstdint>
#include <string>
#include <vector>

namespace TileXR {
namespace checker {

enum class EventKind { RankStart, RankEnd, Copy, Read, Write, FlagStore, FlagWait, PipeSet, PipeWait, Barrier, Diagnostic };
enum class BufferRole { None, UserInput, UserOutput, CommFlag, CommData, LocalSmem, Metadata, RegisteredBuffer };

struct Event {
    uint64_t id = 0;
    EventKind kind = EventKind::Diagnostic;
    int rank = -1;           // who performed it
    int peer = -1;           // owner of the memory touched (or the rank whose flag is awaited)
    int server = 0;
    int peerServer = 0;
    int block = 0;
    BufferRole role = BufferRole::None;
    int64_t slot = -1;       // flag slot or data region id
    int pipe = -1;           // mbarrier / bulk-group id for PipeSet / PipeWait
    int64_t magic = 0;       // (epoch << 32) | value for flag events, epoch for data events
    uint64_t offset = 0;
    uint64_t bytes = 0;
    bool allowFutureProducer = false;
    bool satisfied = true;   // FlagWait / PipeWait: whether the wait completed
    std::string source;      // "file:line" of the modelled protocol step
    std::string detail;
};

enum class FindingKind {
    DEADLOCK,
    FLAG_STALE_MAGIC,
    FLAG_NO_PRODUCER,
    READ_BEFORE_COPY,
    READ_BEFORE_WRITE,
    PIPE_WAIT_NO_PRODUCER,
    DIRECT_PEER_USER_BUFFER,
    OUTPUT_MISMATCH,
    UNSUPPORTED_API,
    EVENT_COVERAGE_GAP,
    BUFFER_LIFETIME,
    AMBIGUOUS_SOURCE,   // two ranks wrote overlapping bytes of one window region in one launch: what a reader finds depends on timing
};
const char *FindingName(FindingKind k);
const char *EventKindName(EventKind k);
const char *RoleName(BufferRole r);

struct Finding {
    FindingKind kind;
    bool fatal = false;
    int rank = -1;
    int peer = -1;
    int64_t slot = -1;
    uint64_t eventId = 0;
    std::string message;
};

struct Injection {
    bool readBeforeCopy = false;     // a consumer reads its window before waiting for the flag
    bool staleMagic = false;         // a producer tags a flag with the previous epoch
    bool missingFlag = false;        // a producer never raises one flag
    bool peerUserRead = false;       // a consumer reads a peer's user buffer directly
    bool pipeWait = false;           // a wait on a pipe (mbarrier) nobody armed
    bool deadlock = false;           // two ranks wait for each other before producing
    bool skipReuseGuard = false;     // a launch overwrites a half a slow peer still reads
    bool corruptOutput = false;      // one output word is flipped
    bool skipEntryMeeting = false;   // zero-copy: a producer writes a peer's own tensor before that peer entered the launch
    bool sharedSlice = false;        // the last rank stores its first tile into rank 0's slice of rank 1's window (3+ ranks)
};

struct CheckerCase {
    std::string op = "allgather";    // allgather | allreduce | alltoall | ep_dispatch | ep_combine
    int rankSize = 2;
    int serverCount = 1;
    int64_t count = 1024;            // int32 elements per rank (collectives)
    int tileElems = 256;
    int64_t bs = 8, h = 16, topK = 2, moeExpertNum = 4;
    std::string scheduler = "round_robin";   // serial | round_robin
    int64_t magic = 1;
    int launches = 1;                // consecutive launches (exercises ping-pong and the reuse guard)
    bool zeroCopy = false;           // allgather: tiles go straight into the peers' registered output tensors, behind an entry meeting
    Injection inject;
};

struct Report {
    CheckerCase testCase;
    std::vector<Event> events;
    std::vector<Finding> findings;
    bool outputsMatch = true;
    bool completed = true;           // every rank reached RankEnd
    std::string Summary() const;
    std::string Json() const;
    bool Passed() const { return findings.empty() && outputsMatch && completed; }
};

// Runs the case (simulation + ordering analysis + oracle comparison).
Report RunCase(const CheckerCase &c);

// Ordering analysis of an event log alone (used for traces captured elsewhere).
std::vector<Finding> CheckOrdering(const std::vector<Event> &events);

// One JSON object per line -> events; malformed lines are reported as UNSUPPORTED_API findings.
std::vector<Event> ParseTraceJsonl(const std::string &text, std::vector<Finding> *problems);
std::string EventsToJsonl(const std::vector<Event> &events);

int WriteReportFiles(const Report &r, const std::string &dir);   // summary.txt + checker_report.json

} // namespace checker
} // namespace TileXR

#endif
