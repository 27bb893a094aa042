#include "checker.h"

#include <algorithm>
#include <array>
#include <memory>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <functional>
#include <map>
#include <set>
#include <sstream>
#include <tuple>
#include <sys/stat.h>

namespace TileXR {
namespace checker {

const char *FindingName(FindingKind k)
{
    switch (k) {
        case FindingKind::DEADLOCK: return "DEADLOCK";
        case FindingKind::FLAG_STALE_MAGIC: return "FLAG_STALE_MAGIC";
        case FindingKind::FLAG_NO_PRODUCER: return "FLAG_NO_PRODUCER";
        case FindingKind::READ_BEFORE_COPY: return "READ_BEFORE_COPY";
        case FindingKind::READ_BEFORE_WRITE: return "READ_BEFORE_WRITE";
        case FindingKind::PIPE_WAIT_NO_PRODUCER: return "PIPE_WAIT_NO_PRODUCER";
        case FindingKind::DIRECT_PEER_USER_BUFFER: return "DIRECT_PEER_USER_BUFFER";
        case FindingKind::OUTPUT_MISMATCH: return "OUTPUT_MISMATCH";
        case FindingKind::UNSUPPORTED_API: return "UNSUPPORTED_API";
        case FindingKind::EVENT_COVERAGE_GAP: return "EVENT_COVERAGE_GAP";
        case FindingKind::BUFFER_LIFETIME: return "BUFFER_LIFETIME";
        case FindingKind::AMBIGUOUS_SOURCE: return "AMBIGUOUS_SOURCE";
    }
    return "UNKNOWN";
}

const char *EventKindName(EventKind k)
{
    static const char *names[] = {"RankStart", "RankEnd", "Copy", "Read", "Write", "FlagStore", "FlagWait", "PipeSet", "PipeWait", "Barrier", "Diagnostic"};
    return names[static_cast<int>(k)];
}

const char *RoleName(BufferRole r)
{
    static const char *names[] = {"none", "user_input", "user_output", "comm_flag", "comm_data", "local_smem", "metadata", "registered_comm_buffer"};
    return names[static_cast<int>(r)];
}

namespace {

constexpr int64_t FLAGS_PER_PAIR = 1024;
constexpr int64_t SLOT_DONE_BASE = 1 << 20;      // done-epoch words, one per source rank
constexpr int64_t SLOT_COUNT = FLAGS_PER_PAIR - 1;

uint64_t MakeFlag(int64_t epoch, int64_t value) { return (static_cast<uint64_t>(epoch) << 32) | static_cast<uint32_t>(value); }

// ---- simulated world ---------------------------------------------------------------------------------

struct RankState {
    std::vector<int32_t> input, output;
    std::map<int64_t, uint64_t> flags;                               // slot -> value, in this rank's window
    std::map<std::pair<int, int64_t>, std::vector<int32_t>> data;    // (half, region) -> words
    size_t pc = 0;
    bool done = false;
};

struct World {
    const CheckerCase &c;
    std::vector<RankState> ranks;
    std::vector<Event> events;
    explicit World(const CheckerCase &cc) : c(cc), ranks(cc.rankSize) {}
    int ServerOf(int rank) const { return rank * c.serverCount / c.rankSize; }
    Event &Log(EventKind kind, int rank, int peer, BufferRole role, int64_t slot, int64_t magic, uint64_t offset, uint64_t bytes,
               const char *source)
    {
        Event e;
        e.id = events.size();
        e.kind = kind;
        e.rank = rank;
        e.peer = peer;
        e.server = ServerOf(rank);
        e.peerServer = peer >= 0 ? ServerOf(peer) : 0;
        e.role = role;
        e.slot = slot;
        e.magic = magic;
        e.offset = offset;
        e.bytes = bytes;
        e.source = source;
        events.push_back(e);
        return events.back();
    }
};

// One step of a rank's program; returns false when it cannot proceed yet (a wait).
typedef std::function<bool(World &, int)> Step;

struct Program {
    std::vector<Step> steps;
};

Step CopyToPeer(int peer, int64_t region, int64_t epoch, uint64_t dstOff, std::function<std::vector<int32_t>(World &, int)> words,
                BufferRole role, const char *src)
{
    return [=](World &w, int rank) {
        const std::vector<int32_t> v = words(w, rank);
        std::vector<int32_t> &dst = w.ranks[peer].data[{static_cast<int>(epoch & 1), region}];
        if (dst.size() < dstOff + v.size()) dst.resize(dstOff + v.size(), 0);
        std::copy(v.begin(), v.end(), dst.begin() + dstOff);
        w.Log(EventKind::Copy, rank, peer, role, region, epoch, dstOff * 4, v.size() * 4, src);
        return true;
    };
}

// Zero-copy: the words land in the peer's own (registered) output tensor, not in its window.
Step CopyToPeerOutput(int peer, int64_t epoch, uint64_t dstOff, std::function<std::vector<int32_t>(World &, int)> words, const char *src)
{
    return [=](World &w, int rank) {
        const std::vector<int32_t> v = words(w, rank);
        std::vector<int32_t> &dst = w.ranks[peer].output;
        if (dst.size() < dstOff + v.size()) dst.resize(dstOff + v.size(), 0);
        std::copy(v.begin(), v.end(), dst.begin() + dstOff);
        w.Log(EventKind::Copy, rank, peer, BufferRole::RegisteredBuffer, 0, epoch, dstOff * 4, v.size() * 4, src);
        return true;
    };
}

Step StoreFlag(int peer, int64_t slot, int64_t epoch, int64_t value, const char *src)
{
    return [=](World &w, int rank) {
        uint64_t &f = w.ranks[peer].flags[slot];
        f = std::max(f, MakeFlag(epoch, value));   // a release store of a monotone flag
        w.Log(EventKind::FlagStore, rank, peer, BufferRole::CommFlag, slot, static_cast<int64_t>(MakeFlag(epoch, value)), 0, 8, src);
        return true;
    };
}

// Logs the wait once (satisfied or not); a blocked wait is retried by the scheduler.
Step WaitFlag(int producer, int64_t slot, int64_t epoch, int64_t value, const char *src)
{
    auto logged = std::make_shared<int64_t>(-1);
    return [=](World &w, int rank) {
        const uint64_t want = MakeFlag(epoch, value);
        auto it = w.ranks[rank].flags.find(slot);
        const bool ok = it != w.ranks[rank].flags.end() && it->second >= want;
        if (*logged < 0) {
            Event &e = w.Log(EventKind::FlagWait, rank, producer, BufferRole::CommFlag, slot, static_cast<int64_t>(want), 0, 8, src);
            e.satisfied = ok;
            *logged = static_cast<int64_t>(e.id);
        } else if (ok) {
            w.events[*logged].satisfied = true;
        }
        return ok;
    };
}

Step ReadWindow(int64_t region, int64_t epoch, uint64_t off, uint64_t words, std::function<void(World &, int, const std::vector<int32_t> &)> sink,
                const char *src)
{
    return [=](World &w, int rank) {
        std::vector<int32_t> &d = w.ranks[rank].data[{static_cast<int>(epoch & 1), region}];
        std::vector<int32_t> v(words, 0);
        for (uint64_t i = 0; i < words && off + i < d.size(); ++i) v[i] = d[off + i];
        w.Log(EventKind::Read, rank, rank, BufferRole::CommData, region, epoch, off * 4, words * 4, src);
        sink(w, rank, v);
        return true;
    };
}

int32_t Pattern(int rank, int64_t i, int launch) { return static_cast<int32_t>(rank * 1000003 + i * 7 + launch * 131); }

void AddGuard(Program &p, const CheckerCase &c, int rank, int64_t epoch)
{
    if (epoch < 3 || c.inject.skipReuseGuard) return;
    for (int peer = 0; peer < c.rankSize; ++peer) {
        if (peer != rank) p.steps.push_back(WaitFlag(peer, SLOT_DONE_BASE + peer, epoch - 2, 0, "tilexr_sync.cuh:KernelPrologue"));
    }
}

void AddDone(Program &p, const CheckerCase &c, int rank, int64_t epoch)
{
    for (int peer = 0; peer < c.rankSize; ++peer) {
        p.steps.push_back(StoreFlag(peer, SLOT_DONE_BASE + rank, epoch, 0, "tilexr_sync.cuh:PublishDone"));
    }
}

// ---- programs -------------------------------------------------------------------------------------------

Program BuildCollective(const CheckerCase &c, int rank)
{
    Program p;
    const int R = c.rankSize;
    const bool gather = c.op == "allgather";
    const bool reduce = c.op == "allreduce";
    const int64_t perPeer = gather || reduce ? c.count : c.count / R;   // words a pair moves
    const int64_t tiles = (perPeer + c.tileElems - 1) / c.tileElems;
    p.steps.push_back([](World &w, int r) { w.Log(EventKind::RankStart, r, -1, BufferRole::None, -1, 0, 0, 0, "launch"); return true; });
    for (int launch = 0; launch < c.launches; ++launch) {
        const int64_t epoch = c.magic + launch;
        p.steps.push_back([=](World &w, int r) {
            RankState &s = w.ranks[r];
            const int64_t nIn = (c.op == "alltoall") ? c.count : c.count;
            s.input.resize(nIn);
            for (int64_t i = 0; i < nIn; ++i) s.input[i] = Pattern(r, i, launch);
            s.output.assign(gather ? c.count * w.c.rankSize : c.count, 0);
            return true;
        });
        AddGuard(p, c, rank, epoch);
        const bool direct = gather && c.zeroCopy;
        if (direct) {
            // every rank announces that it has entered the launch; a producer writes a peer's tensor only after that peer's
            // announcement (its earlier stream work, which may still read the tensor, is finished by then)
            for (int i = 1; i < R; ++i) p.steps.push_back(StoreFlag((rank + i) % R, rank * FLAGS_PER_PAIR + FLAGS_PER_PAIR - 2, epoch, 1, "coll_kernels.cu:announce entry"));
            for (int i = 1; i < R; ++i) {
                const int peer = (rank + i) % R;
                if (c.inject.skipEntryMeeting && rank == 0 && peer == 1) continue;
                p.steps.push_back(WaitFlag(peer, peer * FLAGS_PER_PAIR + FLAGS_PER_PAIR - 2, epoch, 1, "coll_kernels.cu:wait for the peer's entry"));
            }
        }
        if (c.inject.deadlock && launch == 0 && rank < 2) {
            // both ranks wait for the other's first tile before producing their own
            p.steps.push_back(WaitFlag(1 - rank, (1 - rank) * FLAGS_PER_PAIR, epoch, 1, "injected: wait before produce"));
        }
        for (int64_t t = 0; t < tiles; ++t) {
            const int64_t off = t * c.tileElems;
            const int64_t n = std::min<int64_t>(c.tileElems, perPeer - off);
            for (int i = 1; i < R; ++i) {
                const int peer = (rank + i) % R;
                const int64_t srcOff = (gather || reduce) ? off : peer * perPeer + off;
                auto tile = [=](World &w, int r) {
                    const std::vector<int32_t> &in = w.ranks[r].input;
                    return std::vector<int32_t>(in.begin() + srcOff, in.begin() + srcOff + n);
                };
                if (direct) p.steps.push_back(CopyToPeerOutput(peer, epoch, static_cast<uint64_t>(rank) * c.count + off, tile, "coll_kernels.cu:PushBody (zero copy)"));
                else {
                    const bool stray = c.inject.sharedSlice && R >= 3 && rank == R - 1 && peer == 1 && t == 0 && launch == 0;
                    p.steps.push_back(CopyToPeer(peer, stray ? 0 : rank, epoch, off, tile, BufferRole::CommData, "coll_kernels.cu:PushBody"));
                }
                const bool skip = c.inject.missingFlag && rank == 0 && peer == 1 && t == 0 && launch == 0;
                if (!skip) {
                    const int64_t tag = (c.inject.staleMagic && rank == 0 && peer == 1 && t == 0 && launch == 0) ? epoch - 1 : epoch;
                    p.steps.push_back(StoreFlag(peer, rank * FLAGS_PER_PAIR + t, tag, t + 1, "coll_kernels.cu:RaiseTileFlag"));
                }
            }
            if (gather) {
                p.steps.push_back([=](World &w, int r) {
                    RankState &s = w.ranks[r];
                    std::copy(s.input.begin() + off, s.input.begin() + off + n, s.output.begin() + r * c.count + off);
                    return true;
                });
            } else if (c.op == "alltoall") {
                p.steps.push_back([=](World &w, int r) {
                    RankState &s = w.ranks[r];
                    std::copy(s.input.begin() + r * perPeer + off, s.input.begin() + r * perPeer + off + n, s.output.begin() + r * perPeer + off);
                    return true;
                });
            }
        }
        for (int64_t t = 0; t < tiles; ++t) {
            const int64_t off = t * c.tileElems;
            const int64_t n = std::min<int64_t>(c.tileElems, perPeer - off);
            if (reduce) {
                p.steps.push_back([=](World &w, int r) {
                    RankState &s = w.ranks[r];
                    std::copy(s.input.begin() + off, s.input.begin() + off + n, s.output.begin() + off);
                    return true;
                });
            }
            for (int i = 1; i < R; ++i) {
                const int src = (rank + i) % R;
                const bool early = c.inject.readBeforeCopy && rank == 1 && src == 0 && t == 0 && launch == 0;
                Step wait = WaitFlag(src, src * FLAGS_PER_PAIR + t, epoch, t + 1, "coll_kernels.cu:WaitTileFlag");
                Step read = ReadWindow(src, epoch, off, n, [=](World &w, int r, const std::vector<int32_t> &v) {
                    RankState &s = w.ranks[r];
                    for (int64_t j = 0; j < n; ++j) {
                        if (gather) s.output[src * c.count + off + j] = v[j];
                        else if (reduce) s.output[off + j] += v[j];
                        else s.output[src * perPeer + off + j] = v[j];
                    }
                }, "coll_kernels.cu:consumer");
                if (c.inject.peerUserRead && rank == 1 && src == 0 && t == 0 && launch == 0) {
                    p.steps.push_back([=](World &w, int r) {
                        w.Log(EventKind::Read, r, src, BufferRole::UserInput, 0, epoch, off * 4, n * 4, "injected: read of a peer's user buffer");
                        return true;
                    });
                }
                if (direct) {
                    p.steps.push_back(wait);          // the tile is in the output already: its flag is all there is to wait for
                } else if (early) {
                    p.steps.push_back(read);
                    p.steps.push_back(wait);
                } else {
                    p.steps.push_back(wait);
                    p.steps.push_back(read);
                }
            }
        }
        if (c.inject.pipeWait && rank == 0 && launch == 0) {
            p.steps.push_back([](World &w, int r) {
                Event &e = w.Log(EventKind::PipeWait, r, r, BufferRole::LocalSmem, -1, 0, 0, 0, "injected: mbarrier wait without arrive");
                e.pipe = 3;
                e.satisfied = false;
                return true;
            });
        } else if (rank == 0 && launch == 0) {
            p.steps.push_back([](World &w, int r) {
                Event &a = w.Log(EventKind::PipeSet, r, r, BufferRole::LocalSmem, -1, 0, 0, 0, "tilexr_local_copy.cuh:MbarExpectTx");
                a.pipe = 3;
                Event &b = w.Log(EventKind::PipeWait, r, r, BufferRole::LocalSmem, -1, 0, 0, 0, "tilexr_local_copy.cuh:MbarWait");
                b.pipe = 3;
                return true;
            });
        }
        AddDone(p, c, rank, epoch);
    }
    p.steps.push_back([](World &w, int r) { w.Log(EventKind::RankEnd, r, -1, BufferRole::None, -1, 0, 0, 0, "exit"); return true; });
    return p;
}

int ExpertOf(const CheckerCase &c, int rank, int64_t token, int64_t k) { return static_cast<int>((token * c.topK + k * 3 + rank) % c.moeExpertNum); }

// Rows received by `dst` in expert-major, source-major, source order.
std::vector<std::array<int, 4>> EpRows(const CheckerCase &c, int dst)
{
    std::vector<std::array<int, 4>> rows;
    const int per = static_cast<int>(c.moeExpertNum) / c.rankSize;
    for (int le = 0; le < per; ++le) {
        const int e = dst * per + le;
        for (int s = 0; s < c.rankSize; ++s) {
            for (int64_t t = 0; t < c.bs; ++t) {
                for (int64_t k = 0; k < c.topK; ++k) {
                    if (ExpertOf(c, s, t, k) == e) rows.push_back({s, static_cast<int>(t), static_cast<int>(k), e});
                }
            }
        }
    }
    return rows;
}

Program BuildEp(const CheckerCase &c, int rank)
{
    Program p;
    const int R = c.rankSize;
    const int per = static_cast<int>(c.moeExpertNum) / R;
    const int64_t epoch = c.magic;
    const bool combine = c.op == "ep_combine";
    constexpr int64_t REGION_ROWS = 900, REGION_COUNTS = 901;
    p.steps.push_back([](World &w, int r) { w.Log(EventKind::RankStart, r, -1, BufferRole::None, -1, 0, 0, 0, "launch"); return true; });
    if (!combine) {
        // counts to everybody, then rows to their final position, then one flag per destination
        p.steps.push_back([=](World &w, int r) {
            w.ranks[r].output.assign(c.bs * R * c.topK * c.h, 0);
            return true;
        });
        for (int i = 0; i < R; ++i) {
            const int peer = (rank + i) % R;
            p.steps.push_back(CopyToPeer(peer, REGION_COUNTS, epoch, static_cast<uint64_t>(rank) * c.moeExpertNum, [=](World &, int r) {
                std::vector<int32_t> cnt(c.moeExpertNum, 0);
                for (int64_t t = 0; t < c.bs; ++t) {
                    for (int64_t k = 0; k < c.topK; ++k) cnt[ExpertOf(c, r, t, k)]++;
                }
                return cnt;
            }, BufferRole::Metadata, "ep_kernels.cu:publish counts"));
            p.steps.push_back(StoreFlag(peer, rank * FLAGS_PER_PAIR + SLOT_COUNT, epoch, 1, "ep_kernels.cu:count flag"));
        }
        for (int s = 0; s < R; ++s) p.steps.push_back(WaitFlag(s, s * FLAGS_PER_PAIR + SLOT_COUNT, epoch, 1, "ep_kernels.cu:wait counts"));
        for (int dst = 0; dst < R; ++dst) {
            const std::vector<std::array<int, 4>> rows = EpRows(c, dst);
            for (size_t i = 0; i < rows.size(); ++i) {
                if (rows[i][0] != rank) continue;
                const int token = rows[i][1];
                p.steps.push_back(CopyToPeer(dst, REGION_ROWS, epoch, i * c.h, [=](World &, int r) {
                    std::vector<int32_t> v(c.h);
                    for (int64_t j = 0; j < c.h; ++j) v[j] = Pattern(r, token * c.h + j, 0);
                    return v;
                }, BufferRole::CommData, "ep_kernels.cu:send row"));
            }
            const bool skip = c.inject.missingFlag && rank == 0 && dst == 1;
            if (!skip) p.steps.push_back(StoreFlag(dst, rank * FLAGS_PER_PAIR, epoch, 1, "ep_kernels.cu:block flag"));
        }
        const std::vector<std::array<int, 4>> mine = EpRows(c, rank);
        if (c.inject.readBeforeCopy && rank == 1) {
            p.steps.push_back(ReadWindow(REGION_ROWS, epoch, 0, c.h, [](World &, int, const std::vector<int32_t> &) {}, "injected: early window read"));
        }
        for (int s = 0; s < R; ++s) p.steps.push_back(WaitFlag(s, s * FLAGS_PER_PAIR, epoch, 1, "ep_kernels.cu:wait block flags"));
        p.steps.push_back(ReadWindow(REGION_ROWS, epoch, 0, mine.size() * c.h, [=](World &w, int r, const std::vector<int32_t> &v) {
            std::copy(v.begin(), v.end(), w.ranks[r].output.begin());
        }, "ep_kernels.cu:copy out"));
        (void)per;
    } else {
        // every received row goes back to slot (token, k) of its source; the source sums K rows
        p.steps.push_back([=](World &w, int r) {
            w.ranks[r].output.assign(c.bs * c.h, 0);
            return true;
        });
        const std::vector<std::array<int, 4>> mine = EpRows(c, rank);
        bool skippedOne = false;
        for (size_t i = 0; i < mine.size(); ++i) {
            const int src = mine[i][0], token = mine[i][1], k = mine[i][2];
            const int64_t slot = static_cast<int64_t>(token) * c.topK + k;
            p.steps.push_back(CopyToPeer(src, REGION_ROWS, epoch, slot * c.h, [=](World &, int) {
                std::vector<int32_t> v(c.h);
                for (int64_t j = 0; j < c.h; ++j) v[j] = Pattern(src, token * c.h + j, 0) + k;   // "expert" adds k
                return v;
            }, BufferRole::CommData, "ep_kernels.cu:return row"));
            const bool skip = c.inject.missingFlag && rank == 0 && src == 1 && !skippedOne;
            skippedOne = skippedOne || skip;
            if (!skip) p.steps.push_back(StoreFlag(src, 2 * FLAGS_PER_PAIR * 128 + slot, epoch, 1, "ep_kernels.cu:slot flag"));
        }
        for (int64_t t = 0; t < c.bs; ++t) {
            for (int64_t k = 0; k < c.topK; ++k) {
                const int64_t slot = t * c.topK + k;
                const int owner = ExpertOf(c, rank, t, k) / per;
                p.steps.push_back(WaitFlag(owner, 2 * FLAGS_PER_PAIR * 128 + slot, epoch, 1, "ep_kernels.cu:wait slot"));
                p.steps.push_back(ReadWindow(REGION_ROWS, epoch, slot * c.h, c.h, [=](World &w, int r, const std::vector<int32_t> &v) {
                    for (int64_t j = 0; j < c.h; ++j) w.ranks[r].output[t * c.h + j] += v[j];
                }, "ep_kernels.cu:reduce"));
            }
        }
    }
    AddDone(p, c, rank, epoch);
    p.steps.push_back([](World &w, int r) { w.Log(EventKind::RankEnd, r, -1, BufferRole::None, -1, 0, 0, 0, "exit"); return true; });
    return p;
}

// ---- oracle ------------------------------------------------------------------------------------------------

void CompareOutputs(const CheckerCase &c, World &w, Report *rep)
{
    const int R = c.rankSize;
    const int lastLaunch = c.launches - 1;
    for (int r = 0; r < R; ++r) {
        const std::vector<int32_t> &out = w.ranks[r].output;
        std::vector<int32_t> want;
        if (c.op == "allgather") {
            for (int s = 0; s < R; ++s) {
                for (int64_t i = 0; i < c.count; ++i) want.push_back(Pattern(s, i, lastLaunch));
            }
        } else if (c.op == "allreduce") {
            for (int64_t i = 0; i < c.count; ++i) {
                int32_t acc = 0;
                for (int s = 0; s < R; ++s) acc += Pattern(s, i, lastLaunch);
                want.push_back(acc);
            }
        } else if (c.op == "alltoall") {
            const int64_t per = c.count / R;
            for (int s = 0; s < R; ++s) {
                for (int64_t i = 0; i < per; ++i) want.push_back(Pattern(s, r * per + i, lastLaunch));
            }
        } else if (c.op == "ep_dispatch") {
            for (const auto &row : EpRows(c, r)) {
                for (int64_t j = 0; j < c.h; ++j) want.push_back(Pattern(row[0], row[1] * c.h + j, 0));
            }
        } else if (c.op == "ep_combine") {
            for (int64_t t = 0; t < c.bs; ++t) {
                for (int64_t j = 0; j < c.h; ++j) {
                    int32_t acc = 0;
                    for (int64_t k = 0; k < c.topK; ++k) acc += Pattern(r, t * c.h + j, 0) + static_cast<int32_t>(k);
                    want.push_back(acc);
                }
            }
        }
        for (size_t i = 0; i < want.size(); ++i) {
            const int32_t got = i < out.size() ? out[i] : 0;
            if (got != want[i]) {
                rep->outputsMatch = false;
                Finding f;
                f.kind = FindingKind::OUTPUT_MISMATCH;
                f.rank = r;
                std::ostringstream os;
                os << "rank " << r << " element " << i << ": expected " << want[i] << ", got " << got;
                f.message = os.str();
                rep->findings.push_back(f);
                break;
            }
        }
    }
}

void JsonEscape(std::ostringstream &os, const std::string &s)
{
    for (char ch : s) {
        if (ch == '"' || ch == '\\') os << '\\' << ch;
        else if (ch == '\n') os << "\\n";
        else os << ch;
    }
}

} // namespace

// ---- ordering analysis ----------------------------------------------------------------------------------------

std::vector<Finding> CheckOrdering(const std::vector<Event> &events)
{
    std::vector<Finding> out;
    auto add = [&](FindingKind k, const Event &e, const std::string &msg, bool fatal = false) {
        Finding f;
        f.kind = k;
        f.fatal = fatal;
        f.rank = e.rank;
        f.peer = e.peer;
        f.slot = e.slot;
        f.eventId = e.id;
        f.message = msg + " [" + e.source + "]";
        out.push_back(f);
    };
    // unmatched waits
    std::vector<const Event *> unmatched;
    for (const Event &w : events) {
        if (w.kind != EventKind::FlagWait) continue;
        bool matched = false, stale = false;
        for (const Event &s : events) {
            if (s.kind != EventKind::FlagStore || s.rank != w.peer || s.peer != w.rank || s.slot != w.slot) continue;
            if (static_cast<uint64_t>(s.magic) >= static_cast<uint64_t>(w.magic)) matched = true;
            else if ((static_cast<uint64_t>(s.magic) >> 32) + 1 == (static_cast<uint64_t>(w.magic) >> 32) &&
                     (static_cast<uint64_t>(s.magic) & 0xffffffffu) >= (static_cast<uint64_t>(w.magic) & 0xffffffffu)) stale = true;
        }
        if (matched) continue;
        unmatched.push_back(&w);
        if (stale) add(FindingKind::FLAG_STALE_MAGIC, w, "the producer tagged this flag with the previous epoch; the wait can never complete");
        else add(FindingKind::FLAG_NO_PRODUCER, w, "no store ever satisfies this wait");
    }
    for (size_t i = 0; i < unmatched.size(); ++i) {
        for (size_t j = i + 1; j < unmatched.size(); ++j) {
            const Event &a = *unmatched[i], &b = *unmatched[j];
            if (a.rank == b.peer && a.peer == b.rank) {
                add(FindingKind::DEADLOCK, a, "ranks " + std::to_string(a.rank) + " and " + std::to_string(b.rank) + " wait for each other", true);
            }
        }
    }
    // reads need an earlier producer of the same epoch covering the range
    for (const Event &r : events) {
        if (r.kind != EventKind::Read) continue;
        if ((r.role == BufferRole::UserInput || r.role == BufferRole::UserOutput) && r.peer != r.rank) {
            add(FindingKind::DIRECT_PEER_USER_BUFFER, r, "a peer's user buffer was read directly; only windows and registered regions are peer visible");
            continue;
        }
        if (r.role != BufferRole::CommData && r.role != BufferRole::RegisteredBuffer) continue;
        // coverage by the union of earlier copies into the same (owner, region, epoch)
        std::vector<std::pair<uint64_t, uint64_t>> spans;
        for (const Event &p : events) {
            if (p.id >= r.id && !r.allowFutureProducer) break;
            if ((p.kind != EventKind::Copy && p.kind != EventKind::Write) || p.peer != r.peer || p.slot != r.slot || p.magic != r.magic) continue;
            spans.push_back({p.offset, p.offset + p.bytes});
        }
        // Being later in this interleaving is luck; the reader must have WAITED for each producer.
        // Each overlapping copy by another rank must be followed (in that rank's order) by a flag
        // store that a wait of the reader, issued before this read, matches.
        for (const Event &p : events) {
            if (p.id >= r.id) break;
            if ((p.kind != EventKind::Copy && p.kind != EventKind::Write) || p.peer != r.peer || p.slot != r.slot || p.magic != r.magic ||
                p.rank == r.rank || p.offset >= r.offset + r.bytes || p.offset + p.bytes <= r.offset) {
                continue;
            }
            bool ordered = false;
            for (const Event &w : events) {
                if (w.id >= r.id || ordered) break;
                if (w.kind != EventKind::FlagWait || w.rank != r.rank || w.peer != p.rank || w.slot >= SLOT_DONE_BASE) continue;
                for (const Event &st : events) {
                    if (st.id <= p.id || st.kind != EventKind::FlagStore) continue;
                    if (st.rank == p.rank && st.peer == r.rank && st.slot == w.slot &&
                        static_cast<uint64_t>(st.magic) >= static_cast<uint64_t>(w.magic)) {
                        ordered = true;
                        break;
                    }
                }
            }
            if (!ordered) {
                add(r.role == BufferRole::CommData ? FindingKind::READ_BEFORE_COPY : FindingKind::READ_BEFORE_WRITE, r,
                    "read of data produced by rank " + std::to_string(p.rank) + " without first waiting for a flag that rank raised after the copy");
                break;
            }
        }
        std::sort(spans.begin(), spans.end());
        uint64_t covered = r.offset;
        for (const auto &s : spans) {
            if (s.first <= covered && s.second > covered) covered = s.second;
        }
        if (r.bytes > 0 && covered < r.offset + r.bytes) {
            add(r.role == BufferRole::CommData ? FindingKind::READ_BEFORE_COPY : FindingKind::READ_BEFORE_WRITE, r,
                "bytes [" + std::to_string(covered) + ", " + std::to_string(r.offset + r.bytes) + ") were read before any producer of this epoch wrote them");
        }
    }
    // pipes
    for (const Event &w : events) {
        if (w.kind != EventKind::PipeWait) continue;
        bool armed = false;
        for (const Event &s : events) {
            if (s.id >= w.id) break;
            if (s.kind == EventKind::PipeSet && s.rank == w.rank && s.block == w.block && s.pipe == w.pipe) armed = true;
        }
        if (!armed) add(FindingKind::PIPE_WAIT_NO_PRODUCER, w, "wait on a pipe (mbarrier / bulk group) that nobody armed");
    }
    // window reuse: a copy of epoch m >= 3 into a peer needs an earlier successful wait for that peer's done epoch >= m-2
    std::set<std::pair<int, int>> reported;
    for (const Event &c : events) {
        if (c.kind != EventKind::Copy || c.role != BufferRole::CommData || c.peer == c.rank || c.magic < 3) continue;
        bool guarded = false;
        for (const Event &w : events) {
            if (w.id >= c.id) break;
            if (w.kind == EventKind::FlagWait && w.rank == c.rank && w.peer == c.peer && w.slot == SLOT_DONE_BASE + c.peer && w.satisfied &&
                (static_cast<uint64_t>(w.magic) >> 32) + 2 >= static_cast<uint64_t>(c.magic)) {
                guarded = true;
            }
        }
        if (!guarded && reported.insert({c.rank, c.peer}).second) {
            add(FindingKind::BUFFER_LIFETIME, c, "data half reused without checking that the peer finished the launch two epochs ago");
        }
    }
    // a peer's own tensor (registered memory, not a window half) may be written only after that peer is known to have
    // entered this launch: an earlier satisfied wait of the writer for a flag that the peer raised in this epoch or later
    std::set<std::pair<int, int>> early;
    for (const Event &c : events) {
        if (c.kind != EventKind::Copy || c.role != BufferRole::RegisteredBuffer || c.peer == c.rank) continue;
        bool met = false;
        for (const Event &w : events) {
            if (w.id >= c.id) break;
            if (w.kind == EventKind::FlagWait && w.rank == c.rank && w.peer == c.peer && w.satisfied && w.slot < SLOT_DONE_BASE &&
                (static_cast<uint64_t>(w.magic) >> 32) >= static_cast<uint64_t>(c.magic)) {
                met = true;
            }
        }
        if (!met && early.insert({c.rank, c.peer}).second) {
            add(FindingKind::BUFFER_LIFETIME, c, "a peer's own tensor was written before that peer was known to have entered this launch (its earlier work may still read it)");
        }
    }
    // two ranks that write overlapping bytes of one region of one owner in one launch: nothing orders the two stores, so the bytes
    // a reader finds depend on timing (every protocol here gives each source its own slice or its own rows)
    {
        struct Span {
            uint64_t begin, end;
            const Event *e;
        };
        std::map<std::tuple<int, int, int64_t, int64_t>, std::vector<Span>> regions;
        for (const Event &c : events) {
            if ((c.kind != EventKind::Copy && c.kind != EventKind::Write) || c.bytes == 0) continue;
            if (c.role != BufferRole::CommData && c.role != BufferRole::RegisteredBuffer) continue;
            regions[std::make_tuple(c.peer, static_cast<int>(c.role), static_cast<int64_t>(c.slot), static_cast<int64_t>(c.magic))].push_back(
                {c.offset, c.offset + c.bytes, &c});
        }
        std::set<std::tuple<int, int, int>> told;
        for (auto &kv : regions) {
            std::vector<Span> &v = kv.second;
            std::sort(v.begin(), v.end(), [](const Span &a, const Span &b) { return a.begin < b.begin; });
            // sweep: the span that reaches furthest so far, per writer; an overlap with another writer's reach is a finding
            std::map<int, uint64_t> reach;
            for (const Span &sp : v) {
                for (const auto &other : reach) {
                    if (other.first != sp.e->rank && other.second > sp.begin &&
                        told.insert(std::make_tuple(std::min(other.first, sp.e->rank), std::max(other.first, sp.e->rank), sp.e->peer)).second) {
                        add(FindingKind::AMBIGUOUS_SOURCE, *sp.e,
                            "ranks " + std::to_string(other.first) + " and " + std::to_string(sp.e->rank) + " both wrote bytes at offset " +
                                std::to_string(sp.begin) + " of rank " + std::to_string(sp.e->peer) + "'s region in one launch");
                    }
                }
                uint64_t &r = reach[sp.e->rank];
                r = std::max(r, sp.end);
            }
        }
    }
    // coverage
    std::map<int, int> starts, ends;
    for (const Event &e : events) {
        if (e.kind == EventKind::RankStart) starts[e.rank]++;
        if (e.kind == EventKind::RankEnd) ends[e.rank]++;
    }
    for (const auto &kv : starts) {
        if (ends[kv.first] != kv.second) {
            Event e;
            e.rank = kv.first;
            e.source = "scheduler";
            add(FindingKind::EVENT_COVERAGE_GAP, e, "rank " + std::to_string(kv.first) + " never reached its end");
        }
    }
    return out;
}

Report RunCase(const CheckerCase &c)
{
    Report rep;
    rep.testCase = c;
    if (c.rankSize < 1 || c.rankSize > 128 || (c.op != "allgather" && c.op != "allreduce" && c.op != "alltoall" && c.op != "ep_dispatch" && c.op != "ep_combine") ||
        (c.op == "alltoall" && c.count % c.rankSize != 0) || (c.op.rfind("ep_", 0) == 0 && c.moeExpertNum % c.rankSize != 0)) {
        Finding f;
        f.kind = FindingKind::UNSUPPORTED_API;
        f.message = "unsupported case: op " + c.op + " on " + std::to_string(c.rankSize) + " ranks";
        rep.findings.push_back(f);
        rep.completed = false;
        return rep;
    }
    World w(c);
    std::vector<Program> programs;
    for (int r = 0; r < c.rankSize; ++r) programs.push_back(c.op.rfind("ep_", 0) == 0 ? BuildEp(c, r) : BuildCollective(c, r));
    const bool serial = c.scheduler == "serial";
    bool progress = true;
    while (progress) {
        progress = false;
        for (int r = 0; r < c.rankSize; ++r) {
            RankState &s = w.ranks[r];
            while (s.pc < programs[r].steps.size()) {
                if (!programs[r].steps[s.pc](w, r)) break;
                ++s.pc;
                progress = true;
                if (!serial) break;     // round robin: one step per turn
            }
        }
    }
    for (int r = 0; r < c.rankSize; ++r) rep.completed = rep.completed && w.ranks[r].pc == programs[r].steps.size();
    if (c.inject.corruptOutput && !w.ranks[0].output.empty()) w.ranks[0].output[0] ^= 1;
    rep.events = w.events;
    rep.findings = CheckOrdering(rep.events);
    if (rep.completed) CompareOutputs(c, w, &rep);
    return rep;
}

std::string Report::Summary() const
{
    std::ostringstream os;
    os << "case: op=" << testCase.op << " ranks=" << testCase.rankSize << " servers=" << testCase.serverCount << " scheduler=" << testCase.scheduler
       << " launches=" << testCase.launches << "\n";
    os << "events: " << events.size() << "  completed: " << (completed ? "yes" : "no") << "  outputs: " << (outputsMatch ? "match" : "MISMATCH") << "\n";
    os << "findings: " << findings.size() << "\n";
    for (const Finding &f : findings) {
        os << "  " << (f.fatal ? "FATAL " : "") << FindingName(f.kind) << " rank " << f.rank << " peer " << f.peer << " slot " << f.slot << ": " << f.message << "\n";
    }
    os << (Passed() ? "RESULT: PASS\n" : "RESULT: FAIL\n");
    return os.str();
}

std::string Report::Json() const
{
    std::ostringstream os;
    os << "{\"op\": \"" << testCase.op << "\", \"rank_size\": " << testCase.rankSize << ", \"server_count\": " << testCase.serverCount
       << ", \"scheduler\": \"" << testCase.scheduler << "\", \"launches\": " << testCase.launches << ", \"events\": " << events.size()
       << ", \"completed\": " << (completed ? "true" : "false") << ", \"outputs_match\": " << (outputsMatch ? "true" : "false")
       << ", \"passed\": " << (Passed() ? "true" : "false") << ", \"findings\": [";
    for (size_t i = 0; i < findings.size(); ++i) {
        const Finding &f = findings[i];
        os << (i ? ", " : "") << "{\"kind\": \"" << FindingName(f.kind) << "\", \"fatal\": " << (f.fatal ? "true" : "false") << ", \"rank\": " << f.rank
           << ", \"peer\": " << f.peer << ", \"slot\": " << f.slot << ", \"event\": " << f.eventId << ", \"message\": \"";
        JsonEscape(os, f.message);
        os << "\"}";
    }
    os << "]}";
    return os.str();
}

std::string EventsToJsonl(const std::vector<Event> &events)
{
    std::ostringstream os;
    for (const Event &e : events) {
        os << "{\"id\": " << e.id << ", \"kind\": \"" << EventKindName(e.kind) << "\", \"rank\": " << e.rank << ", \"peer\": " << e.peer
           << ", \"block\": " << e.block << ", \"role\": \"" << RoleName(e.role) << "\", \"slot\": " << e.slot << ", \"pipe\": " << e.pipe
           << ", \"magic\": " << e.magic << ", \"offset\": " << e.offset << ", \"bytes\": " << e.bytes << ", \"satisfied\": " << (e.satisfied ? 1 : 0)
           << ", \"source\": \"";
        JsonEscape(os, e.source);
        os << "\"}\n";
    }
    return os.str();
}

namespace {
bool FindInt(const std::string &line, const char *key, int64_t *out)
{
    const std::string k = std::string("\"") + key + "\":";
    size_t p = line.find(k);
    if (p == std::string::npos) return false;
    p += k.size();
    while (p < line.size() && line[p] == ' ') ++p;
    char *end = nullptr;
    const long long v = std::strtoll(line.c_str() + p, &end, 10);
    if (end == line.c_str() + p) return false;
    *out = v;
    return true;
}
bool FindStr(const std::string &line, const char *key, std::string *out)
{
    const std::string k = std::string("\"") + key + "\":";
    size_t p = line.find(k);
    if (p == std::string::npos) return false;
    p = line.find('"', p + k.size());
    if (p == std::string::npos) return false;
    const size_t q = line.find('"', p + 1);
    if (q == std::string::npos) return false;
    *out = line.substr(p + 1, q - p - 1);
    return true;
}
} // namespace

std::vector<Event> ParseTraceJsonl(const std::string &text, std::vector<Finding> *problems)
{
    std::vector<Event> out;
    std::istringstream is(text);
    std::string line;
    int lineNo = 0;
    bool allHaveIds = true;
    while (std::getline(is, line)) {
        ++lineNo;
        if (line.find_first_not_of(" \t\r") == std::string::npos) continue;
        Event e;
        std::string kind, role;
        int64_t v = 0;
        bool good = FindStr(line, "kind", &kind) && FindInt(line, "rank", &v);
        if (good) {
            e.rank = static_cast<int>(v);
            good = false;
            for (int k = 0; k <= static_cast<int>(EventKind::Diagnostic); ++k) {
                if (kind == EventKindName(static_cast<EventKind>(k))) {
                    e.kind = static_cast<EventKind>(k);
                    good = true;
                }
            }
        }
        if (!good) {
            if (problems != nullptr) {
                Finding f;
                f.kind = FindingKind::UNSUPPORTED_API;
                f.message = "trace line " + std::to_string(lineNo) + " is not a recognised event";
                problems->push_back(f);
            }
            continue;
        }
        // Files of several ranks concatenate into one trace: when every line carries its global id, the events are put
        // in that order below; otherwise the line order is the order.
        if (FindInt(line, "id", &v)) e.id = static_cast<uint64_t>(v);
        else allHaveIds = false;
        if (FindInt(line, "peer", &v)) e.peer = static_cast<int>(v);
        if (FindInt(line, "block", &v)) e.block = static_cast<int>(v);
        if (FindInt(line, "slot", &v)) e.slot = v;
        if (FindInt(line, "pipe", &v)) e.pipe = static_cast<int>(v);
        if (FindInt(line, "magic", &v)) e.magic = v;
        if (FindInt(line, "offset", &v)) e.offset = static_cast<uint64_t>(v);
        if (FindInt(line, "bytes", &v)) e.bytes = static_cast<uint64_t>(v);
        if (FindInt(line, "satisfied", &v)) e.satisfied = v != 0;
        if (FindStr(line, "role", &role)) {
            for (int r = 0; r <= static_cast<int>(BufferRole::RegisteredBuffer); ++r) {
                if (role == RoleName(static_cast<BufferRole>(r))) e.role = static_cast<BufferRole>(r);
            }
        }
        FindStr(line, "source", &e.source);
        out.push_back(e);
    }
    if (allHaveIds) {
        std::stable_sort(out.begin(), out.end(), [](const Event &a, const Event &b) { return a.id < b.id; });
    }
    for (size_t i = 0; i < out.size(); ++i) out[i].id = i;
    return out;
}

int WriteReportFiles(const Report &r, const std::string &dir)
{
    mkdir(dir.c_str(), 0755);
    std::ofstream a(dir + "/summary.txt"), b(dir + "/checker_report.json"), t(dir + "/events.jsonl");
    if (!a || !b || !t) return -1;
    a << r.Summary();
    b << r.Json() << "\n";
    t << EventsToJsonl(r.events);
    return 0;
}

} // namespace checker
} // namespace TileXR
