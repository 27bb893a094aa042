// tilexr_checker: command-line front end of the protocol checker.
//
//   tilexr_checker --op allgather --ranks 4 --servers 2 --count 4096 --tile 512 --launches 3
//       --scheduler round_robin --out report_dir [--inject-read-before-copy] ...
//   tilexr_checker --trace events.jsonl            # analyse a captured event trace
//
// Exit code 0 when the case passes, 1 when there are findings, 2 on bad usage.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>

#include "checker.h"

using namespace TileXR::checker;

static void Usage()
{
    std::puts("usage: tilexr_checker [--op allgather|allreduce|alltoall|ep_dispatch|ep_combine] [--ranks N] [--servers N]\n"
              "       [--count N] [--tile N] [--bs N] [--h N] [--topk N] [--experts N] [--launches N] [--magic N]\n"
              "       [--scheduler serial|round_robin] [--out DIR] [--trace FILE]\n"
              "       [--inject-read-before-copy] [--inject-stale-magic] [--inject-missing-flag] [--inject-peer-user-read]\n"
              "       [--inject-pipe-wait] [--inject-deadlock] [--inject-skip-reuse-guard] [--inject-corrupt-output]\n"
              "       [--zero-copy] [--inject-skip-entry-meeting] [--inject-shared-slice]");
}

int main(int argc, char **argv)
{
    CheckerCase c;
    std::string out, trace;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        auto next = [&](const char *name) -> const char * {
            if (i + 1 >= argc) {
                std::fprintf(stderr, "%s needs a value\n", name);
                std::exit(2);
            }
            return argv[++i];
        };
        if (a == "--op") c.op = next("--op");
        else if (a == "--ranks") c.rankSize = std::atoi(next("--ranks"));
        else if (a == "--servers") c.serverCount = std::atoi(next("--servers"));
        else if (a == "--count") c.count = std::atoll(next("--count"));
        else if (a == "--tile") c.tileElems = std::atoi(next("--tile"));
        else if (a == "--bs") c.bs = std::atoll(next("--bs"));
        else if (a == "--h") c.h = std::atoll(next("--h"));
        else if (a == "--topk") c.topK = std::atoll(next("--topk"));
        else if (a == "--experts") c.moeExpertNum = std::atoll(next("--experts"));
        else if (a == "--launches") c.launches = std::atoi(next("--launches"));
        else if (a == "--magic") c.magic = std::atoll(next("--magic"));
        else if (a == "--scheduler") c.scheduler = next("--scheduler");
        else if (a == "--out") out = next("--out");
        else if (a == "--trace") trace = next("--trace");
        else if (a == "--inject-read-before-copy") c.inject.readBeforeCopy = true;
        else if (a == "--inject-stale-magic") c.inject.staleMagic = true;
        else if (a == "--inject-missing-flag") c.inject.missingFlag = true;
        else if (a == "--inject-peer-user-read") c.inject.peerUserRead = true;
        else if (a == "--inject-pipe-wait") c.inject.pipeWait = true;
        else if (a == "--inject-deadlock") c.inject.deadlock = true;
        else if (a == "--inject-skip-reuse-guard") c.inject.skipReuseGuard = true;
        else if (a == "--inject-corrupt-output") c.inject.corruptOutput = true;
        else if (a == "--inject-shared-slice") c.inject.sharedSlice = true;
        else if (a == "--inject-skip-entry-meeting") c.inject.skipEntryMeeting = true;
        else if (a == "--zero-copy") c.zeroCopy = true;
        else if (a == "--help" || a == "-h") {
            Usage();
            return 0;
        } else {
            std::fprintf(stderr, "unknown argument %s\n", a.c_str());
            Usage();
            return 2;
        }
    }
    Report rep;
    if (!trace.empty()) {
        std::ifstream f(trace);
        if (!f) {
            std::fprintf(stderr, "cannot read %s\n", trace.c_str());
            return 2;
        }
        std::stringstream ss;
        ss << f.rdbuf();
        std::vector<Finding> problems;
        rep.events = ParseTraceJsonl(ss.str(), &problems);
        rep.findings = CheckOrdering(rep.events);
        rep.findings.insert(rep.findings.end(), problems.begin(), problems.end());
        rep.testCase.op = "trace";
    } else {
        rep = RunCase(c);
    }
    std::fputs(rep.Summary().c_str(), stdout);
    if (!out.empty() && WriteReportFiles(rep, out) != 0) {
        std::fprintf(stderr, "cannot write report files under %s\n", out.c_str());
        return 2;
    }
    return rep.Passed() ? 0 : 1;
}
