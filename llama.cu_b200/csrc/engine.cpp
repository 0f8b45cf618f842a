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
    uint64_t draws = 0;        // random numbers drawn for this session so far (seeded sampling)
};

// a finished conversation parked for prefix reuse == an entry of CacheManager::caches
// (xtask/src/service/cache_manager.rs:9-12): its token history and the KV sequence that holds it
struct Parked {
    std::vector<uint32_t> history;
    int seq;
};

// counter-based generator: the k-th random number of session `id` under `seed` depends on nothing else, so a
// sampled conversation is reproducible whatever it is batched with (the reference draws rand::random() per row)
inline float seeded_uniform(uint64_t seed, uint64_t id, uint64_t k) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ull * (id + 1) + 0xBF58476D1CE4E5B9ull * (k + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) * (1.0f / 16777216.0f);  // 24 bits -> [0, 1)
}

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
    // token budget of a round and largest prefill chunk (0: the reference's behaviour — whole prompts, no budget)
    uint32_t max_round_tokens = 0, prefill_chunk = 0;
    // prefix reuse
    std::map<uint64_t, Parked> parked;  // insertion order == the reference's BTreeMap<Instant, _>
    uint64_t park_clock = 0;
    int next_fake_seq = 0;              // sequence labels when there is no context (host-only use)
    // seeded sampling
    bool seeded = false;
    uint64_t seed = 0;
    std::vector<float> randoms;
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

// Token budget and chunked prefill — what the reference leaves as a TODO (exec/engine_manager.rs:83,100-109: a round
// takes whole prompts and the engine asserts at most 1024 tokens, exec/engine.rs:68).  max_round_tokens > 0: a round
// holds at most that many tokens; every decoding session always gets its one token, prompts share what is left in
// session order.  prefill_chunk > 0: no prompt contributes more than that per round.  A prompt that is not finished
// in a round contributes a chunk whose entry in the round's `output` list is LCU_ENGINE_NO_OUTPUT (its sampled pair
// is to be ignored) and costs no step of max_steps.  0 / 0 (default): whole prompts, as the reference.
int lcu_engine_set_budget(lcu_engine *e, uint32_t max_round_tokens, uint32_t prefill_chunk) {
    ENGINE_REQUIRE(e, "engine_set_budget: null engine");
    e->max_round_tokens = max_round_tokens;
    e->prefill_chunk = prefill_chunk;
    return LCU_OK;
}

// == `EngineManager::prepare` (exec/engine_manager.rs:72-130)
int lcu_engine_prepare(lcu_engine *e, lcu_round_info *info) {
    ENGINE_REQUIRE(e && info, "engine_prepare: null argument");
    e->tokens.clear(); e->fast_map.clear(); e->reqs.clear(); e->sample.clear();
    e->output.clear(); e->finished.clear(); e->overflow.clear();
    std::map<uint64_t, size_t> pre_output;
    pre_output.swap(e->pre_output);
    // tokens left for prompts once every decoding session has its one
    uint64_t budget = ~0ull;
    if (e->max_round_tokens) {
        uint64_t n_decode = 0;
        for (auto &kv : e->all)
            if (kv.second.active && !kv.second.has_prompt) ++n_decode;
        budget = e->max_round_tokens > n_decode ? e->max_round_tokens - n_decode : 0;
    }
    size_t out_idx = 0;
    for (auto &kv : e->all) {  // std::map iterates in id order, like the reference's BTreeMap
        const uint64_t id = kv.first;
        Stub &s = kv.second;
        if (!s.active) continue;
        uint32_t take = s.seq_len;  // tokens of this session in this round
        if (s.has_prompt) {
            if (e->prefill_chunk && take > e->prefill_chunk) take = e->prefill_chunk;
            if ((uint64_t)take > budget) take = (uint32_t)budget;
            if (take == 0) continue;  // no room in this round: the prompt waits
        }
        const uint64_t end = (uint64_t)s.pos + s.seq_len;
        if (end > e->nctx) {  // cache overflow: the session is handed back, nothing is run for it
            e->overflow.push_back(id);
            s.active = false;
            continue;
        }
        const uint32_t pos = s.pos;
        s.pos += take;
        e->sample.push_back(s.args);
        lcu_req rq;
        rq.seq = s.seq;
        rq.pos = pos;
        rq.len = take;
        e->reqs.push_back(rq);
        if (s.has_prompt) {  // prefill: the whole prompt, or its next chunk
            budget -= take;
            e->tokens.insert(e->tokens.end(), s.prompt.begin(), s.prompt.begin() + take);
            if (take < s.seq_len) {  // more of the prompt to come: nothing is sampled, no step is used
                s.prompt.erase(s.prompt.begin(), s.prompt.begin() + take);
                s.seq_len -= take;
                e->output.push_back(LCU_ENGINE_NO_OUTPUT);
                ++out_idx;
                continue;
            }
            s.prompt.clear();
            s.has_prompt = false;
            s.seq_len = 1;
        } else {  // decode: a placeholder the device overwrites with the previous sample
            e->fast_map.push_back((uint32_t)pre_output[id]);
            e->fast_map.push_back((uint32_t)e->tokens.size());
            e->tokens.push_back(0);
        }
        e->output.push_back(id);
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

// ------------------------------------------------------------------ prefix reuse == CacheManager
// (xtask/src/service/cache_manager.rs:22-66)

// == `CacheManager::insert`: a finished session's token history and KV sequence are parked for reuse.
int lcu_engine_cache_insert(lcu_engine *e, uint64_t id, const uint32_t *tokens, uint32_t n) {
    ENGINE_REQUIRE(e && (tokens || n == 0), "engine_cache_insert: null argument");
    auto it = e->all.find(id);
    ENGINE_REQUIRE(it != e->all.end(), "engine_cache_insert: unknown session");
    ENGINE_REQUIRE(!it->second.active, "engine_cache_insert: session is running");
    Parked p;
    p.history.assign(tokens, tokens + n);
    p.seq = it->second.seq;
    e->parked[e->park_clock++] = p;
    e->pre_output.erase(id);
    e->all.erase(it);
    return LCU_OK;
}

// == `CacheManager::send`: a new session for `tokens` starts from the parked cache that shares the longest prefix with
// tokens[0 .. n-1) (the latest parked one among equals — Iterator::max_by_key keeps the last maximum; with NO common
// prefix a parked cache is still taken and restarted at 0, as the reference does), rolled back to that length; without
// parked caches a fresh sequence.  Only tokens[pos ..] are run.  reused_out: the number of tokens not recomputed.
int lcu_engine_cache_send(lcu_engine *e, const uint32_t *tokens, uint32_t n, const lcu_sample_args *args, int max_steps,
                          uint64_t *id_out, uint32_t *reused_out) {
    ENGINE_REQUIRE(e && tokens && n > 0 && max_steps > 0 && id_out, "engine_cache_send: bad arguments");
    bool found = false;
    uint64_t best_key = 0;
    uint32_t best_len = 0;
    for (auto &kv : e->parked) {
        const std::vector<uint32_t> &h = kv.second.history;
        uint32_t len = 0;
        while (len < h.size() && len + 1 < n && h[len] == tokens[len]) ++len;
        if (!found || len >= best_len) { found = true; best_key = kv.first; best_len = len; }
    }
    int seq;
    uint32_t pos = 0;
    if (found) {
        seq = e->parked[best_key].seq;
        pos = best_len;
        e->parked.erase(best_key);
        if (e->ctx) {  // pages past the kept prefix go back to the pool, as KVCache::update does on a rollback
            int rc = lcu_seq_resize(e->ctx, seq, pos);
            if (rc) return rc;
        }
    } else if (e->ctx) {
        int rc = lcu_seq_create(e->ctx, &seq);
        if (rc) return rc;
    } else {
        seq = e->next_fake_seq++;
    }
    int rc = lcu_engine_session_new(e, seq, args, id_out);
    if (rc) return rc;
    e->all[*id_out].pos = pos;
    if (reused_out) *reused_out = pos;
    return lcu_engine_start(e, *id_out, tokens + pos, n - pos, max_steps);
}

int lcu_engine_cache_count(const lcu_engine *e) { return e ? (int)e->parked.size() : 0; }

// ------------------------------------------------------------------ seeded sampling
// With a seed the engine draws the per-request random numbers itself: the k-th number of a session depends only on
// (seed, session id, k).  The reference's host draws rand::random() per row and step (exec/output_head.rs:111) and
// cannot be replayed.
int lcu_engine_set_seed(lcu_engine *e, uint64_t seed) {
    ENGINE_REQUIRE(e, "engine_set_seed: null engine");
    e->seeded = true;
    e->seed = seed;
    return LCU_OK;
}

// Draws the random numbers of the prepared round (one per request; 0 for arg-max rows and unfinished prefill
// chunks) and advances the sessions' draw counters: what lcu_engine_step does under a seed, for hosts that call
// lcu_step themselves.  Call once per prepared round.
int lcu_engine_draw_randoms(lcu_engine *e) {
    ENGINE_REQUIRE(e && e->seeded, "engine_draw_randoms: no seed set");
    e->randoms.assign(e->reqs.size(), 0.f);
    for (size_t i = 0; i < e->reqs.size(); ++i) {
        const lcu_sample_args &a = e->sample[i];
        if (e->output[i] == LCU_ENGINE_NO_OUTPUT || a.temperature == 0.f || a.top_k == 1) continue;
        Stub &st = e->all[e->output[i]];
        e->randoms[i] = seeded_uniform(e->seed, e->output[i], st.draws++);
    }
    return LCU_OK;
}

// the numbers of the last lcu_engine_draw_randoms / seeded lcu_engine_step
const float *lcu_engine_round_randoms(const lcu_engine *e) { return e && e->seeded ? e->randoms.data() : nullptr; }

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
    if (e->seeded) {
        rc = lcu_engine_draw_randoms(e);
        if (rc) return rc;
        randoms = e->randoms.data();
    }
    return lcu_step(e->ctx, stream, info->n_req, e->reqs.data(), e->tokens.data(), any_sampling ? e->sample.data() : nullptr,
                    any_sampling ? randoms : nullptr, e->fast_map.empty() ? nullptr : e->fast_map.data(), info->n_fast,
                    out_dev);
}

}  // extern "C"
