// TEST INFRASTRUCTURE — drives the reference's own generation loop, mako::gen::Session (src/gen/session.cpp,
// compiled unmodified from the reference checkout), over a stand-in engine, and prints what it generates. Built twice
// by oracle/Makefile from this one source:
//   _ref/session_dropin_ref    with the reference's src/gen/sampler.{hpp,cpp}: the CPU sampler;
//   _ref/session_dropin_mako   with oracle/dropin/shim/gen/sampler.hpp first on the include path and
//                              libmako_b200.so on the link line: the same loop on the B200 sampler.
// A test runs both and compares the outputs line by line: same seeds, same logits -> the same tokens, the same
// numbers of drafts made and kept. The stand-in engine follows the pattern of the reference's own session tests
// (a gen::Model that records its tokens, tests/session_respell_test.cpp:31-78), with logits that depend on the
// context so that sampling, penalties and draft verification all have something to decide.
//
// Scenarios (the three decode loops of Session::run):
//   plain        one token a step: sample() + accept()                      (src/gen/session.cpp:522-547, else branch)
//   drafter      multi-token drafts, verify() row by row, keep()            (src/gen/session.cpp:451-506)
//   mtp          one-token drafts in two-token steps, verify(), rollback()  (src/gen/session.cpp:509-540)
//   forced       every third token forced by the caller: no draw consumed   (src/gen/session.cpp:441-444, 481-484)
#include "gen/session.hpp"

#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace {

constexpr uint32_t kVocab = 40000;

// A small PCG (XSH-RR 64/32) for the stand-in engine's logits.
struct Pcg {
    uint64_t state, inc;
    Pcg(uint64_t seed, uint64_t seq) : state(0), inc((seq << 1) | 1)
    {
        next();
        state += seed;
        next();
    }
    uint32_t next()
    {
        const uint64_t old = state;
        state = old * 6364136223846793005ull + inc;
        const uint32_t xs = uint32_t(((old >> 18) ^ old) >> 27), rot = uint32_t(old >> 59);
        return (xs >> rot) | (xs << ((32 - rot) & 31));
    }
    float uniform() { return float(next() >> 8) * (1.0f / 16777216.0f); }
};

uint64_t mix(uint64_t h, uint64_t v)
{
    h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    return h;
}

// Logits after a context: a broad background, a few strong tokens that depend on the last two tokens of the context.
void logits_after(const std::vector<int32_t>& ctx, size_t len, std::vector<float>& out)
{
    uint64_t h = 0x1234;
    for (size_t i = len >= 2 ? len - 2 : 0; i < len; ++i)
        h = mix(h, uint64_t(ctx[i]) + 1);
    Pcg g(h, 77);
    out.resize(kVocab);
    for (uint32_t i = 0; i < kVocab; i += 2) { // Box-Muller
        const float u1 = (float(g.next() >> 8) + 1.0f) * (1.0f / 16777216.0f), u2 = g.uniform();
        const float r = 2.0f * std::sqrt(-2.0f * std::log(u1));
        out[i] = r * std::cos(6.2831853f * u2);
        if (i + 1 < kVocab)
            out[i + 1] = r * std::sin(6.2831853f * u2);
    }
    for (int k = 0; k < 6; ++k) // strong tokens among the low ids, so that repeats (and their penalties) happen
        out[g.next() % 300] = 8.0f + 6.0f * g.uniform();
}

int32_t argmax(const std::vector<float>& l, size_t off = 0)
{
    int32_t best = 0;
    for (uint32_t i = 1; i < kVocab; ++i)
        if (l[off + i] > l[off + best])
            best = int32_t(i);
    return best;
}

class Engine : public mako::gen::Model {
public:
    enum Kind { plain, drafter, mtp };
    explicit Engine(Kind k) : kind_(k) {}
    std::vector<int32_t> ctx;

    const std::vector<float>& step(int32_t token) override
    {
        ctx.push_back(token);
        logits_after(ctx, ctx.size(), row_);
        return row_;
    }
    const std::vector<float>& prefill(std::span<const int32_t> tokens, const std::function<bool()>&,
                                      const std::function<void(size_t)>&) override
    {
        ctx.insert(ctx.end(), tokens.begin(), tokens.end());
        logits_after(ctx, ctx.size(), row_);
        return row_;
    }
    uint32_t position() const override { return uint32_t(ctx.size()); }
    uint32_t max_context() const override { return 4096; }
    uint32_t n_vocab() const override { return kVocab; }
    void reset() override { ctx.clear(); }
    Checkpoint checkpoint() override
    {
        Checkpoint c;
        c.pos = position();
        c.state.resize(ctx.size() * 4);
        std::memcpy(c.state.data(), ctx.data(), c.state.size());
        return c;
    }
    void restore(const Checkpoint& c) override
    {
        ctx.resize(c.pos);
        std::memcpy(ctx.data(), c.state.data(), c.state.size());
    }
    std::vector<std::byte> save_positions(uint32_t) const override { return {}; }
    void load_positions(uint32_t, std::span<const std::byte>) override {}
    uint32_t checkpoint_slots() const override { return 4; }

    // one-token drafter: the most likely token after `next` (a guess the sampler accepts with its probability)
    bool has_mtp() const override { return kind_ == mtp; }
    int32_t mtp_draft(int32_t next) override
    {
        std::vector<int32_t> c = ctx;
        c.push_back(next);
        std::vector<float> l;
        logits_after(c, c.size(), l);
        return argmax(l);
    }
    int32_t mtp_draft(std::span<const int32_t> next) override { return mtp_draft(next.back()); }
    const std::vector<float>& step2(int32_t a, int32_t b) override
    {
        ctx.push_back(a);
        std::vector<float> first;
        logits_after(ctx, ctx.size(), first);
        ctx.push_back(b);
        std::vector<float> second;
        logits_after(ctx, ctx.size(), second);
        two_ = first;
        two_.insert(two_.end(), second.begin(), second.end());
        return two_;
    }
    void rollback() override { ctx.pop_back(); }

    // multi-token drafter: three greedy guesses after `next`
    bool has_drafter() const override { return kind_ == drafter; }
    std::vector<int32_t> draft(int32_t next) override
    {
        std::vector<int32_t> c = ctx, out;
        c.push_back(next);
        std::vector<float> l;
        for (int i = 0; i < 3; ++i) {
            logits_after(c, c.size(), l);
            out.push_back(argmax(l));
            c.push_back(out.back());
        }
        return out;
    }
    const std::vector<float>& verify(std::span<const int32_t> tokens) override
    {
        rows_.clear();
        verified_ = ctx.size();
        std::vector<float> l;
        for (int32_t t : tokens) {
            ctx.push_back(t);
            logits_after(ctx, ctx.size(), l);
            rows_.insert(rows_.end(), l.begin(), l.end());
        }
        return rows_;
    }
    void keep(uint32_t n) override { ctx.resize(verified_ + n); }

private:
    Kind kind_;
    size_t verified_ = 0;
    std::vector<float> row_, two_, rows_;
};

void run(const char* name, Engine::Kind kind, const mako::gen::SamplingParams& sp, uint64_t seed, bool force_some)
{
    Engine e(kind);
    mako::gen::Session s(e);
    mako::gen::GenerateParams p;
    p.sampling = sp;
    p.seed = seed;
    p.max_tokens = 96;
    p.speculative = kind != Engine::plain;
    p.lookup_match = 0;
    size_t asked = 0;
    if (force_some)
        p.forced = [&asked](const float* logits) -> int32_t {
            return (++asked % 3 == 0) ? int32_t(logits[7] > logits[9] ? 7 : 9) : -1;
        };
    const std::vector<int32_t> prompt = {11, 22, 33, 44};
    const mako::gen::GenerateResult r = s.generate(prompt, p);
    std::printf("%s finish=%d drafts=%u accepted=%u tokens=", name, int(r.finish), r.drafts, r.accepted);
    for (int32_t t : r.tokens)
        std::printf("%d ", t);
    std::printf("\n");
    // a second turn on the same session: the prompt continues the context (tokens reused, a fresh sampler)
    std::vector<int32_t> again(s.context().begin(), s.context().end());
    again.push_back(55);
    const mako::gen::GenerateResult r2 = s.generate(again, p);
    std::printf("%s/turn2 reused=%u tokens=", name, r2.reused_tokens);
    for (int32_t t : r2.tokens)
        std::printf("%d ", t);
    std::printf("\n");
}

} // namespace

int main()
{
    mako::gen::SamplingParams warm; // temperature 1, everything else off
    mako::gen::SamplingParams pen;
    pen.temperature = 0.8f;
    pen.top_p = 0.9f;
    pen.min_p = 0.05f;
    pen.repetition_penalty = 1.1f;
    pen.presence_penalty = 0.5f;
    pen.frequency_penalty = 0.3f;
    mako::gen::SamplingParams nucleus;
    nucleus.temperature = 0.7f;
    nucleus.top_k = 40;
    nucleus.top_p = 0.95f;
    mako::gen::SamplingParams greedy;
    greedy.temperature = 0.0f;
    try {
        run("plain/penalised", Engine::plain, pen, 1, false);
        run("plain/nucleus", Engine::plain, nucleus, 2, false);
        run("plain/warm", Engine::plain, warm, 3, false);
        run("plain/greedy", Engine::plain, greedy, 4, false);
        run("drafter/penalised", Engine::drafter, pen, 5, false);
        run("drafter/nucleus", Engine::drafter, nucleus, 6, false);
        run("drafter/greedy", Engine::drafter, greedy, 7, false);
        run("mtp/penalised", Engine::mtp, pen, 8, false);
        run("mtp/nucleus", Engine::mtp, nucleus, 9, false);
        run("forced/plain", Engine::plain, pen, 10, true);
        run("forced/drafter", Engine::drafter, pen, 11, true);
    } catch (const std::exception& ex) {
        std::fprintf(stderr, "session_dropin: %s\n", ex.what());
        return 2;
    }
    return 0;
}
