// Host-side round builder: the C++ counterpart of the reference's `EngineManager`
// (llama.cu/src/exec/engine_manager.rs:15-156) and of the `pos` / `out_idx` helpers of its engine
// loop (exec/engine.rs:352-371).  It owns no GPU state: it decides what goes into each round —
// which sessions, which tokens, where the previous samples are fed back on the device — and
// hands the round to lcu_step.  Everything here runs (and is tested) without a GPU.
#include <cstring>
#include <map>
#include <vector>

#include "../../include/lcu.h"

namespace lcu {
void set_error(const char *fmt, ...);
}

namespace {

struct Stub {  // == SessionStub + State (exec/engine.rs:33-66)
    int seq = -1;
    lcu_sample_args args{0.f, 1.f, ~0ull};
    uint32_t pos = 0;          // == DistKVCache::pos
    uint32_t seq_len = 0;      // tokens of the next round
    int remain_steps = 0;
    bool active = false;
    bool has_prompt = false;
    std::vector<uint32_t> prompt;
};

}  // namespace

struct lcu_engine {
    lcu_ctx *ctx = nullptr;
    uint32_t nctx = 0;
    uint64_t next_id = 0;
    std::map<uint64_t, Stub> all;              // every session the caller created
    std::map<uint64_t, size_t> pre_output;     // id -> index of its pair in the previous round
    // the prepared round == Round (exec/engine_manager.rs:22-31)
    std::vector<uint32_t> tokens, fast_map;
    std::vector<lcu_req> reqs;
    std::vector<lcu_sample_args> sample;
    std::vector<uint64_t> output, finished, overflow;
};

#define ENGINE_REQUIRE(cond, ...)        \
    do {                                 \
        if (!(cond)) {                   \
            lcu::set_error(__VA_ARGS__); \
            return LCU_ERR_INVALID;      \
        }                                \
    } while (0)

extern "C" {

int lcu_engine_create(lcu_ctx *ctx, uint32_t nctx, lcu_engine **out) {
    ENGINE_REQUIRE(out && nctx > 0, "engine_create: bad arguments");
    lcu_engine *e = new lcu_engine();
    e->ctx = ctx;
    e->nctx = nctx;
    *out = e;
    return LCU_OK;
}

int lcu_engine_destroy(lcu_engine *e) {
    delete e;
    return LCU_OK;
}

// == creating a `Session{id, sample_args, cache}` (lib.rs / exec/mod.rs:61-69); `seq` is the KV handle
int lcu_engine_session_new(lcu_engine *e, int seq, const lcu_sample_args *args, uint64_t *id_out) {
    ENGINE_REQUIRE(e && id_out, "engine_session_new: null argument");
    Stub s;
    s.seq = seq;
    if (args) {
        // SampleArgs::new (op/random_sample/mod.rs:58-73)
        ENGINE_REQUIRE(args->temperature >= 0.f, "engine_session_new: NegativeTemperature");
        ENGINE_REQUIRE(args->top_k != 0 && args->top_p > 0.f, "engine_session_new: NonPositiveTop");
        s.args = *args;
        if (s.args.top_p > 1.f) s.args.top_p = 1.f;
    }
    *id_out = e->next_id;
    e->all[e->next_id++] = s;
    return LCU_OK;
}

// == `Terminal::start` -> `Command::Insert` (lib.rs:233-243, exec/engine_manager.rs:133-137)
int lcu_engine_start(lcu_engine *e, uint64_t id, const uint32_t *prompt, uint32_t n, int max_steps) {
    ENGINE_REQUIRE(e && prompt && n > 0 && max_steps > 0, "engine_start: bad arguments");
    auto it = e->all.find(id);
    ENGINE_REQUIRE(it != e->all.end(), "engine_start: unknown session");
    Stub &s = it->second;
    s.prompt.assign(prompt, prompt + n);
    s.has_prompt = true;
    s.seq_len = n;
    s.remain_steps = max_steps;
    s.active = true;
    return LCU_OK;
}

// == `Command::Remove` (exec/engine_manager.rs:138-148): the session leaves the batch, keeps its cache
int lcu_engine_remove(lcu_engine *e, uint64_t id) {
    ENGINE_REQUIRE(e, "engine_remove: null engine");
    auto it = e->all.find(id);
    if (it != e->all.end()) it->second.active = false;
    e->pre_output.erase(id);
    return LCU_OK;
}

int lcu_engine_session_pos(const lcu_engine *e, uint64_t id, uint32_t *pos_out) {
    ENGINE_REQUIRE(e && pos_out, "engine_session_pos: null argument");
    auto it = e->all.find(id);
    ENGINE_REQUIRE(it != e->all.end(), "engine_session_pos: unknown session");
    *pos_out = it->second.pos;
    return LCU_OK;
}

// rolls `cache.pos` back (prefix reuse, xtask/src/service/cache_manager.rs:38-55)
int lcu_engine_session_set_pos(lcu_engine *e, uint64_t id, uint32_t pos) {
    ENGINE_REQUIRE(e, "engine_session_set_pos: null engine");
    auto it = e->all.find(id);
    ENGINE_REQUIRE(it != e->all.end(), "engine_session_set_pos: unknown session");
    ENGINE_REQUIRE(!it->second.active, "engine_session_set_pos: session is running");
    it->second.pos = pos;
    return LCU_OK;
}

// == `EngineManager::prepare` (exec/engine_manager.rs:72-130)
int lcu_engine_prepare(lcu_engine *e, lcu_round_info *info) {
    ENGINE_REQUIRE(e && info, "engine_prepare: null argument");
    e->tokens.clear(); e->fast_map.clear(); e->reqs.clear(); e->sample.clear();
    e->output.clear(); e->finished.clear(); e->overflow.clear();
    std::map<uint64_t, size_t> pre_output;
    pre_output.swap(e->pre_output);
    size_t out_idx = 0;
    for (auto &kv : e->all) {  // std::map iterates in id order, like the reference's BTreeMap
        const uint64_t id = kv.first;
        Stub &s = kv.second;
        if (!s.active) continue;
        const uint64_t end = (uint64_t)s.pos + s.seq_len;
        if (end > e->nctx) {  // cache overflow: the session is handed back, nothing is run for it
            e->overflow.push_back(id);
            s.active = false;
            continue;
        }
        const uint32_t pos = s.pos;
        s.pos = (uint32_t)end;
        e->sample.push_back(s.args);
        e->output.push_back(id);
        lcu_req rq;
        rq.seq = s.seq;
        rq.pos = pos;
        rq.len = s.seq_len;
        e->reqs.push_back(rq);
        if (s.has_prompt) {  // prefill: the whole prompt
            e->tokens.insert(e->tokens.end(), s.prompt.begin(), s.prompt.end());
            s.prompt.clear();
            s.has_prompt = false;
            s.seq_len = 1;
        } else {  // decode: a placeholder the device overwrites with the previous sample
            e->fast_map.push_back((uint32_t)pre_output[id]);
            e->fast_map.push_back((uint32_t)e->tokens.size());
            e->tokens.push_back(0);
        }
        if (--s.remain_steps == 0) {
            e->finished.push_back(id);
            s.active = false;
        } else {
            e->pre_output[id] = out_idx;
        }
        ++out_idx;
    }
    info->n_tok = (int)e->tokens.size();
    info->n_req = (int)e->reqs.size();
    info->n_fast = (int)(e->fast_map.size() / 2);
    info->n_finished = (int)e->finished.size();
    info->n_overflow = (int)e->overflow.size();
    return LCU_OK;
}

const uint32_t *lcu_engine_round_tokens(const lcu_engine *e) { return e ? e->tokens.data() : nullptr; }
const lcu_req *lcu_engine_round_reqs(const lcu_engine *e) { return e ? e->reqs.data() : nullptr; }
const uint32_t *lcu_engine_round_fast_map(const lcu_engine *e) { return e ? e->fast_map.data() : nullptr; }
const lcu_sample_args *lcu_engine_round_sample_args(const lcu_engine *e) { return e ? e->sample.data() : nullptr; }
const uint64_t *lcu_engine_round_output(const lcu_engine *e) { return e ? e->output.data() : nullptr; }
const uint64_t *lcu_engine_round_finished(const lcu_engine *e) { return e ? e->finished.data() : nullptr; }
const uint64_t *lcu_engine_round_overflow(const lcu_engine *e) { return e ? e->overflow.data() : nullptr; }

// `pos()` and `out_idx()` of the engine loop (exec/engine.rs:352-371) for the prepared round
int lcu_engine_round_positions(const lcu_engine *e, uint32_t *pos_out, uint32_t *out_idx_out) {
    ENGINE_REQUIRE(e, "engine_round_positions: null engine");
    uint32_t itok = 0;
    for (size_t r = 0; r < e->reqs.size(); ++r) {
        const lcu_req &q = e->reqs[r];
        for (uint32_t i = 0; i < q.len; ++i)
            if (pos_out) pos_out[itok + i] = q.pos + i;
        if (out_idx_out) out_idx_out[r] = itok + q.len - 1;  // out == 1: the last token of the request
        itok += q.len;
    }
    return LCU_OK;
}

// One iteration of `Worker::lead`'s loop (exec/engine.rs:222-295): prepare, then run the round.
// Returns LCU_OK with info->n_tok == 0 when there is nothing to run.
int lcu_engine_step(lcu_engine *e, lcu_stream_t stream, const float *randoms, lcu_kv_pair *out_dev,
                    lcu_round_info *info) {
    ENGINE_REQUIRE(e && e->ctx && info, "engine_step: null argument or engine without a context");
    int rc = lcu_engine_prepare(e, info);
    if (rc || info->n_tok == 0) return rc;
    bool any_sampling = false;
    for (const lcu_sample_args &a : e->sample)
        if (!(a.temperature == 0.f || a.top_k == 1)) any_sampling = true;
    return lcu_step(e->ctx, stream, info->n_req, e->reqs.data(), e->tokens.data(), any_sampling ? e->sample.data() : nullptr,
                    any_sampling ? randoms : nullptr, e->fast_map.empty() ? nullptr : e->fast_map.data(), info->n_fast,
                    out_dev);
}

}  // extern "C"
