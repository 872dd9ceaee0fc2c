// fsb_request.cpp - request fields and command-line flags -> sampling parameters, with the defaults, aliases and
// range errors of the reference's server (src/server.cpp:1060-1072 of paragontasx/ferro) and CLI (src/main.cpp:250-262).
// Pure host code: no CUDA call, usable before any engine exists.
#include <cstdlib>
#include <cstring>

#include "../../include/ferro_sampler_b200.h"

extern "C" {

void fsb_server_defaults_init(fsb_server_defaults* d) {
    if (!d) return;
    d->repeat_penalty = 0.0f;   // src/server.h: <= 0 means "the sampler's own default"
    d->repeat_last_n = -1;
    d->penalize_prompt = 1;
}

// src/server.cpp:1060-1072.  A field counts only if the request carried it as a JSON number (the reference's jnum
// falls back to the default for anything else): the caller sets its bit in `present` only then.
int fsb_params_from_request(const fsb_request_fields* f, const fsb_server_defaults* d, int32_t prompt_tokens, ferro_sampler_params* out) {
    if (!f || !out || prompt_tokens < 0) return FSB_ERR_INVALID;
    fsb_server_defaults dd;
    if (d) dd = *d;
    else fsb_server_defaults_init(&dd);
    ferro_sampler_params sp;
    fsb_params_default(&sp);
    auto has = [&](unsigned bit) { return (f->present & bit) != 0u; };
    sp.temperature = (float)(has(FSB_REQ_TEMPERATURE) ? f->temperature : (double)sp.temperature);
    sp.top_p = (float)(has(FSB_REQ_TOP_P) ? f->top_p : (double)sp.top_p);
    sp.top_k = (int32_t)(has(FSB_REQ_TOP_K) ? f->top_k : (double)sp.top_k);
    sp.min_p = (float)(has(FSB_REQ_MIN_P) ? f->min_p : (double)sp.min_p);
    const double server_pen = dd.repeat_penalty > 0 ? (double)dd.repeat_penalty : (double)sp.repetition_penalty;
    sp.repetition_penalty = (float)(has(FSB_REQ_REPETITION_PENALTY) ? f->repetition_penalty : has(FSB_REQ_REPEAT_PENALTY) ? f->repeat_penalty : server_pen);
    sp.repeat_last_n = (int32_t)(has(FSB_REQ_REPEAT_LAST_N) ? f->repeat_last_n : has(FSB_REQ_PENALTY_LAST_N) ? f->penalty_last_n : (double)dd.repeat_last_n);
    const bool pen_prompt = has(FSB_REQ_PENALIZE_PROMPT) ? f->penalize_prompt != 0 : dd.penalize_prompt != 0;
    if (!pen_prompt) sp.penalty_from = prompt_tokens;   // penalty scope "generated": the window never reaches into the prompt
    sp.seed = (uint64_t)(has(FSB_REQ_SEED) ? f->seed : 0.0);
    if (sp.temperature < 0 || sp.top_p <= 0 || sp.top_p > 1 || sp.top_k < 0 || sp.repetition_penalty <= 0 || sp.repeat_last_n < -1)
        return FSB_ERR_RANGE;   // the reference answers 400 "sampling parameter out of range"
    *out = sp;
    return FSB_OK;
}

// src/main.cpp:250-262: the flags that reach the sampler.  `p` takes the generate command's flags, `d` the server's.
int fsb_params_apply_cli_flag(ferro_sampler_params* p, fsb_server_defaults* d, const char* flag, const char* value) {
    if (!p || !d || !flag) return FSB_ERR_INVALID;
    static const char* const kFlags[] = {"--temp", "--top-k", "--top-p", "--min-p", "--rep-penalty", "--seed", "--repeat-penalty",
                                         "--repeat-last-n", "--penalty-scope"};
    int which = -1;
    for (int i = 0; i < (int)(sizeof kFlags / sizeof kFlags[0]); ++i)
        if (std::strcmp(flag, kFlags[i]) == 0) which = i;
    if (which < 0) return 0;               // not a sampling flag
    if (!value) return FSB_ERR_INVALID;    // the reference exits with "<flag> needs a value"
    switch (which) {
        case 0: p->temperature = (float)std::atof(value); break;
        case 1: p->top_k = std::atoi(value); break;
        case 2: p->top_p = (float)std::atof(value); break;
        case 3: p->min_p = (float)std::atof(value); break;
        case 4: p->repetition_penalty = (float)std::atof(value); break;
        case 5: p->seed = (uint64_t)std::atoll(value); break;
        case 6: d->repeat_penalty = (float)std::atof(value); break;
        case 7:
            d->repeat_last_n = std::atoi(value);
            p->repeat_last_n = d->repeat_last_n;
            break;
        case 8:
            if (std::strcmp(value, "all") != 0 && std::strcmp(value, "generated") != 0) return FSB_ERR_RANGE;   // "--penalty-scope must be all or generated"
            d->penalize_prompt = std::strcmp(value, "all") == 0 ? 1 : 0;
            break;
    }
    return 1;
}

}  // extern "C"
