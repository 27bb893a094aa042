// Turns one launch's stage statistics into trace.json / summary.csv / analysis.md /
// report.html (+ ai_prompt.md).  File set follows the reference's per-launch report
// (src/collectives/host/perf_trace_report.h:14-45).
#include <algorithm>
#include <fstream>
#include <iomanip>
#include <sstream>

#include "perf_trace_session.h"
#include "tilexr_types.h"

namespace TileXR {

std::vector<PerfStageSummary> SummarizeLaunch(const PerfLaunchRecord &rec)
{
    std::vector<PerfStageSummary> out;
    const uint32_t stages = rec.header.stageCount;
    const uint32_t div = rec.header.cycleToUsDivisor;
    for (uint32_t s = 0; s < stages; ++s) {
        PerfStageSummary sum{};
        sum.stageId = s;
        sum.name = s < TILEXR_PERF_STAGE_COUNT ? TILEXR_PERF_STAGE_TABLE[s].name : "stage";
        uint64_t first = ~0ull, last = 0;
        for (uint32_t c = 0; c < rec.header.maxCoreCount; ++c) {
            const TileXRPerfCoreStageStats &st = rec.stats[TileXRPerfStatsIndex(c, s, stages)];
            if (st.count == 0) continue;
            sum.count += st.count;
            sum.sumUs += TileXRPerfTicksToUs(st.sumCycles, div);
            const double mx = TileXRPerfTicksToUs(st.sumCycles, div);
            if (mx > sum.maxUs) {
                sum.maxUs = mx;
                sum.maxCore = c;
            }
            first = std::min(first, st.firstStartCycle);
            last = std::max(last, st.lastEndCycle);
            sum.bytes += st.aux0;
        }
        sum.spanUs = (sum.count > 0 && last >= first) ? TileXRPerfTicksToUs(last - first, div) : 0.0;
        out.push_back(sum);
    }
    return out;
}

std::string AnalyzeLaunch(const PerfLaunchRecord &rec, const std::vector<PerfStageSummary> &summary)
{
    std::ostringstream os;
    const PerfStageSummary *total = nullptr;
    const PerfStageSummary *worst = nullptr;
    for (const PerfStageSummary &s : summary) {
        if (s.stageId == TILEXR_PERF_KERNEL_TOTAL) total = &s;
        else if (s.stageId != TILEXR_PERF_CHUNK_TOTAL && (worst == nullptr || s.maxUs > worst->maxUs)) worst = &s;
    }
    os << "# " << TileXROpName(static_cast<int>(rec.info.opType)) << " launch " << rec.launchId << " on rank "
       << rec.info.rank << "/" << rec.info.rankSize << "\n\n";
    os << "- message bytes: " << rec.info.messageBytes << "\n- blocks: " << rec.info.blocks << "\n";
    if (total != nullptr && total->count > 0) {
        os << "- kernel span: " << std::fixed << std::setprecision(2) << total->spanUs << " us\n";
        if (total->spanUs > 0 && rec.info.messageBytes > 0) {
            os << "- algorithm bandwidth: " << (rec.info.messageBytes / total->spanUs / 1000.0) << " GB/s\n";
        }
    }
    if (worst != nullptr && worst->count > 0) {
        os << "- longest stage on a single block: `" << worst->name << "` " << worst->maxUs << " us on block "
           << worst->maxCore << "\n";
        if (worst->stageId == TILEXR_PERF_FLAG_POLL_WAIT) {
            os << "- interpretation: blocks mostly wait for peers' tiles; look at the slowest producer rank or add "
                  "producer blocks.\n";
        } else if (worst->stageId == TILEXR_PERF_LOCAL_INPUT_TO_IPC) {
            os << "- interpretation: pushing tiles over NVLink dominates; the launch is transfer bound.\n";
        } else if (worst->stageId == TILEXR_PERF_PEER_IPC_TO_OUTPUT) {
            os << "- interpretation: copying landed tiles to the output dominates; register the output buffer to "
                  "enable the zero-copy path.\n";
        } else if (worst->stageId == TILEXR_PERF_POST_SYNC) {
            os << "- interpretation: the launch waited for peers to finish an earlier launch (window reuse guard).\n";
        }
    }
    return os.str();
}

int WriteLaunchReport(const std::string &dir, const PerfLaunchRecord &rec, bool emitAiPrompt, const std::string &aiCommand,
                      const std::string &incompleteReason)
{
    const std::vector<PerfStageSummary> summary = SummarizeLaunch(rec);
    const std::string analysis = AnalyzeLaunch(rec, summary);
    {
        std::ofstream f(dir + "/trace.json");
        if (!f) return TILEXR_ERROR_INTERNAL;
        f << "{\n  \"schema\": \"tilexr-perf-trace-v1\",\n  \"op\": \"" << TileXROpName(static_cast<int>(rec.info.opType))
          << "\",\n  \"opType\": " << rec.info.opType << ",\n  \"dataType\": " << rec.info.dataType
          << ",\n  \"rank\": " << rec.info.rank << ",\n  \"rankSize\": " << rec.info.rankSize
          << ",\n  \"launchId\": " << rec.launchId << ",\n  \"messageBytes\": " << rec.info.messageBytes
          << ",\n  \"blocks\": " << rec.info.blocks << ",\n  \"ticksPerUs\": " << rec.header.cycleToUsDivisor
          << ",\n  \"incomplete\": " << (incompleteReason.empty() ? "false" : "true") << ",\n  \"incompleteReason\": \""
          << incompleteReason << "\",\n  \"stages\": [";
        for (uint32_t s = 0; s < TILEXR_PERF_STAGE_COUNT; ++s) {
            f << (s ? ", " : "") << "{\"id\": " << s << ", \"name\": \"" << TILEXR_PERF_STAGE_TABLE[s].name
              << "\", \"category\": " << TILEXR_PERF_STAGE_TABLE[s].category << "}";
        }
        f << "],\n  \"records\": [\n";
        bool firstRec = true;
        for (const TileXRPerfCoreStageStats &st : rec.stats) {
            if (st.count == 0) continue;
            f << (firstRec ? "" : ",\n") << "    {\"rank\": " << st.rank << ", \"core\": " << st.core << ", \"stage\": "
              << st.stageId << ", \"count\": " << st.count << ", \"sum\": " << st.sumCycles << ", \"min\": "
              << st.minCycles << ", \"max\": " << st.maxCycles << ", \"firstStart\": " << st.firstStartCycle
              << ", \"lastEnd\": " << st.lastEndCycle << ", \"bytes\": " << st.aux0 << "}";
            firstRec = false;
        }
        f << "\n  ]\n}\n";
    }
    {
        std::ofstream f(dir + "/summary.csv");
        f << "stage,name,count,sum_us,max_block_us,max_block,span_us,bytes\n";
        for (const PerfStageSummary &s : summary) {
            f << s.stageId << "," << s.name << "," << s.count << "," << s.sumUs << "," << s.maxUs << "," << s.maxCore << ","
              << s.spanUs << "," << s.bytes << "\n";
        }
    }
    {
        std::ofstream f(dir + "/analysis.md");
        f << analysis;
        if (!incompleteReason.empty()) f << "\n**Incomplete report:** " << incompleteReason << "\n";
    }
    {
        std::ofstream f(dir + "/report.html");
        f << "<html><head><meta charset=\"utf-8\"><title>TileXR launch " << rec.launchId
          << "</title><style>td,th{padding:2px 8px;border:1px solid #999}table{border-collapse:collapse}</style></head><body>"
          << "<h2>" << TileXROpName(static_cast<int>(rec.info.opType)) << " &mdash; rank " << rec.info.rank << ", launch "
          << rec.launchId << "</h2><table><tr><th>stage</th><th>count</th><th>sum us</th><th>max block us</th>"
          << "<th>block</th><th>span us</th><th>bytes</th></tr>";
        for (const PerfStageSummary &s : summary) {
            f << "<tr><td>" << s.name << "</td><td>" << s.count << "</td><td>" << s.sumUs << "</td><td>" << s.maxUs
              << "</td><td>" << s.maxCore << "</td><td>" << s.spanUs << "</td><td>" << s.bytes << "</td></tr>";
        }
        f << "</table><pre>" << analysis << "</pre></body></html>\n";
    }
    if (emitAiPrompt) {
        std::ofstream f(dir + "/ai_prompt.md");
        f << "You are looking at the stage profile of one collective kernel launch.\n"
          << "Suggested command (not executed by the library): " << aiCommand << "\n\n"
          << analysis << "\nPer-stage table:\n\n";
        for (const PerfStageSummary &s : summary) {
            f << "- " << s.name << ": count " << s.count << ", sum " << s.sumUs << " us, slowest block " << s.maxCore
              << " with " << s.maxUs << " us\n";
        }
        f << "\nWhich stage bounds this launch, and what would you change first?\n";
    }
    return TILEXR_SUCCESS;
}

} // namespace TileXR
