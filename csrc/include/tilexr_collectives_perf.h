// Stage-profiling sessions for the collectives library (reference:
// src/include/tilexr_collectives_perf.h:8-24).  While a session is active every collective
// launch gets a device trace buffer; WriteReport reads the buffers back and writes, per
// launch, `launch<N>/trace.json`, `summary.csv`, `analysis.md` and `report.html` under
// `<outputDir>/rank<R>/`.
#ifndef TILEXR_COLLECTIVES_PERF_H
#define TILEXR_COLLECTIVES_PERF_H

#ifdef __cplusplus
extern "C" {
#endif

typedef void *TileXRCollectivePerfSession;

typedef struct TileXRCollectivePerfConfig {
    int enabled;
    const char *outputDir;
    unsigned int sampleEveryN;   // profile every N-th launch (0 or 1: all)
    int emitAiPrompt;            // also write ai_prompt.md (a text summary to paste into an assistant)
    const char *aiCommand;       // recorded in ai_prompt.md, never executed
} TileXRCollectivePerfConfig;

int TileXRCollectivePerfSessionCreate(const TileXRCollectivePerfConfig *config, TileXRCollectivePerfSession *session);
int TileXRCollectivePerfSessionDestroy(TileXRCollectivePerfSession session);
int TileXRCollectivePerfSetActiveSession(TileXRCollectivePerfSession session);
int TileXRCollectivePerfWriteReport(TileXRCollectivePerfSession session);
int TileXRCollectivePerfWriteIncompleteReport(TileXRCollectivePerfSession session, const char *reason);

#ifdef __cplusplus
}
#endif

#endif
