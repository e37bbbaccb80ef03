"""The C++ runtime (page table, prefix cache, scheduling policy, step planner, request engine,
streaming, tokenizer, chat template) driven from Python with scripted sessions — no GPU."""
import json

import torch
import threading
import time

import numpy as np
import pytest

from tensorrt_edge_llm_b200.runtime import native as rt


def test_page_table_and_prefix_cache():
    t = rt.KVPageTable(num_pages=10, page_size=4, max_seats=3, max_pages_per_seq=4)
    t.reserve(0, 9)                      # 3 pages
    assert t.capacity_tokens(0) == 12 and t.free_pages == 7
    assert t.take_dirty_rows() == [0] and t.take_dirty_rows() == []
    t.commit(0, 9)
    t.rewind(0, 6)
    assert t.length(0) == 6
    with pytest.raises(RuntimeError):
        t.reserve(0, 17)                 # > 4 pages
    assert not t.can_reserve(1, 40)
    rows = t.rows([0, 1])
    assert rows.shape == (2, 4) and (rows[1] == -1).all() and (rows[0][:3] >= 0).all()
    cache = rt.PrefixCache(t.allocator(), 4, 8)
    toks = list(range(100, 111))         # 11 tokens → 2 full pages reusable (the last token is always computed)
    assert cache.lookup(toks).tokens == 0
    assert cache.insert(toks, 9, t.pages(0)) == 2
    m = cache.lookup(toks)
    assert m.tokens == 8 and m.pages == t.pages(0)[:2]
    t.adopt_prefix(1, m.pages, m.tokens)
    assert t.length(1) == 8 and t.allocator().refcount(m.pages[0]) == 3     # seat 0, cache, seat 1
    t.free_seat(0)
    t.free_seat(1)
    assert t.free_pages == 8             # two pages still held by the cache
    assert cache.evict(5) == 2 and t.free_pages == 10
    assert cache.lookup(toks[:4] + [7] * 7).tokens == 0
    pool = rt.ResidentSlotPool(2)
    a, b = pool.acquire(), pool.acquire()
    assert pool.acquire() == -1 and pool.in_use == 2
    e = pool.epoch(a)
    pool.release(a)
    assert pool.acquire() == a and pool.epoch(a) == e + 1


def _caps(b=4, inp=2048, page=64, compact=True):
    c = rt.SessionCapabilities()
    c.max_batch_size, c.max_input_length, c.kv_page_size, c.compact = b, inp, page, compact
    return c


def test_scheduling_policy_defaults_and_validation():
    caps = _caps(b=8, inp=4096)
    o = rt.SchedulingOptions()
    r = rt.resolve_scheduling_policy(o, caps)
    assert r.mode == rt.IfbSchedulingMode.Mixed
    assert r.max_num_tokens == 576 and r.max_chunk_tokens == 512       # roundUp64(512+8), min(512, roundDown64(576-8))
    assert rt.resolve_scheduling_policy(o, _caps(compact=False)).mode == rt.IfbSchedulingMode.SingleCohort
    o.max_chunk_tokens = 100
    assert "multiple" in rt.validate_scheduling_options(o, caps)
    o.max_chunk_tokens = 128
    o.max_num_tokens = 4
    assert rt.validate_scheduling_options(o, caps) != ""
    o.max_num_tokens = 0
    o.mode = rt.IfbSchedulingMode.Mixed
    assert "compact" in rt.validate_scheduling_options(o, _caps(compact=False))


def _res(slot, prompt, prefilled, generated=0, prio=0, arrival=None):
    s = rt.ResidentState()
    s.slot, s.prompt_len, s.prefilled, s.generated, s.priority = slot, prompt, prefilled, generated, prio
    s.arrival = slot if arrival is None else arrival
    return s


def _planner(mode, max_tokens=256, chunk=128, policy=rt.SchedulingPolicy.Fcfs, preempt=rt.PreemptionMode.NoPreemption):
    lim = rt.StepPlannerLimits()
    lim.max_batch_size, lim.max_input_length, lim.kv_page_size = 8, 4096, 64
    p = rt.ResolvedSchedulingPolicy()
    p.mode, p.policy, p.preemption = mode, policy, preempt
    p.max_num_tokens, p.max_chunk_tokens, p.max_pause_steps = max_tokens, chunk, 2
    return rt.StepPlanner(lim, p)


def test_step_planner_mixed_layout_and_chunking():
    pl = _planner(rt.IfbSchedulingMode.Mixed)
    plan = pl.plan([_res(0, 300, 0), _res(1, 50, 50, generated=3), _res(2, 10, 10, generated=1)])
    kinds = [(s.slot, s.kind, s.start, s.length, s.last_chunk) for s in plan.seqs]
    # context chunks first, decode rows after (compact layout); the chunk is page aligned
    assert kinds[0] == (0, rt.WorkKind.Context, 0, 128, False)
    assert [k[0] for k in kinds[1:]] == [1, 2] and all(k[1] == rt.WorkKind.Decode for k in kinds[1:])
    assert kinds[1][2] == 52 and plan.num_context == 1 and plan.num_decode == 2 and plan.total_tokens == 130
    # the last chunk is not page aligned and is flagged
    plan = pl.plan([_res(0, 300, 256)])
    assert (plan.seqs[0].start, plan.seqs[0].length, plan.seqs[0].last_chunk) == (256, 44, True)
    # budget: two prompts share max_num_tokens, trimmed to page boundaries
    plan = _planner(rt.IfbSchedulingMode.Mixed, max_tokens=200, chunk=192).plan([_res(0, 500, 0), _res(1, 500, 0)])
    assert [s.length for s in plan.seqs] == [192] and plan.total_tokens == 192


def test_step_planner_modes_priority_and_pause():
    res = [_res(0, 100, 100, generated=2), _res(1, 200, 0)]
    plan = _planner(rt.IfbSchedulingMode.PrefillFirst).plan(res)
    assert plan.num_context == 1 and plan.num_decode == 0 and plan.paused == [0]
    plan = _planner(rt.IfbSchedulingMode.SingleCohort, max_tokens=4096).plan(res)
    assert plan.seqs[0].length == 200 and plan.seqs[0].last_chunk and plan.num_decode == 0
    plan = _planner(rt.IfbSchedulingMode.SingleCohort).plan([_res(0, 10, 10, 1), _res(1, 10, 10, 1)])
    assert plan.num_decode == 2
    # priority policy orders context work
    res = [_res(0, 500, 0, prio=0), _res(1, 500, 0, prio=5)]
    plan = _planner(rt.IfbSchedulingMode.Mixed, max_tokens=128, policy=rt.SchedulingPolicy.Priority).plan(res)
    assert plan.seqs[0].slot == 1
    # pause preemption: with a tiny budget decode rows yield room for a page of prefill, then are forced back in
    pl = _planner(rt.IfbSchedulingMode.Mixed, max_tokens=66, chunk=64, preempt=rt.PreemptionMode.Pause)
    res = [_res(i, 8, 8, generated=1) for i in range(4)] + [_res(9, 640, 0)]
    plan = pl.plan(res)
    assert plan.num_context == 1 and plan.seqs[0].length == 64 and plan.num_decode == 2 and len(plan.paused) == 2
    for r in res:
        if r.slot in plan.paused:
            r.paused_steps = 2
    plan2 = pl.plan(res)
    assert all(s in [q.slot for q in plan2.seqs] for s in plan.paused)


class ScriptedSession(rt.RuntimeSession):
    """Echo model: every generated token is prompt[0] + position; finishes on max_tokens via the engine."""

    def __init__(self, batch=2, fail_on_step=None, page=4):
        super().__init__()
        self.batch, self.fail_on_step, self.page = batch, fail_on_step, page
        self.free = list(range(batch))
        self.seqs = {}
        self.steps = 0
        self.plans = []

    def capabilities(self):
        c = rt.SessionCapabilities()
        c.compact, c.max_batch_size, c.max_input_length, c.kv_page_size, c.max_kv_tokens = True, self.batch, 64, self.page, 128
        return c

    def admit(self, request_id, req):
        r = rt.AdmissionResult()
        if len(req.prompt_ids) > 64:
            r.admitted, r.retry_later, r.reason = False, False, "EDGELLM_INPUT_TOO_LONG"
            return r
        if not self.free:
            r.admitted, r.retry_later, r.reason = False, True, "no seat"
            return r
        r.admitted, r.slot = True, self.free.pop(0)
        self.seqs[r.slot] = (list(req.prompt_ids), 0)
        return r

    def execute(self, plan):
        self.steps += 1
        self.plans.append([(s.slot, int(s.kind == rt.WorkKind.Context), s.length) for s in plan.seqs])
        if self.fail_on_step is not None and self.steps == self.fail_on_step:
            raise RuntimeError("injected executor failure")
        out = rt.StepResult()
        deltas = []
        for s in plan.seqs:
            prompt, gen = self.seqs[s.slot]
            if s.kind == rt.WorkKind.Context and not s.last_chunk:
                continue
            d = rt.TokenDelta()
            d.slot, d.tokens = s.slot, [prompt[0] + gen]
            self.seqs[s.slot] = (prompt, gen + 1)
            deltas.append(d)
        out.deltas = deltas
        return out

    def release(self, slot):
        self.seqs.pop(slot, None)
        self.free.append(slot)


def _req(first, n_prompt=6, max_tokens=4, prio=0):
    r = rt.GenerationRequest()
    r.prompt_ids, r.max_tokens, r.priority = [first] * n_prompt, max_tokens, prio
    return r


def test_request_engine_inflight_batching_and_streaming():
    sessions = []

    def factory():
        s = ScriptedSession(batch=2)
        sessions.append(s)
        return s

    cfg = rt.EngineConfig()
    cfg.max_batch_size = 2
    eng = rt.RequestEngine(cfg, factory)
    handles = [eng.submit(_req(100 * (i + 1), max_tokens=3 + i))[0] for i in range(4)]
    outs = [h.get(10.0) for h in handles]
    assert outs[0] == [100, 101, 102] and outs[3] == [400, 401, 402, 403, 404, 405]
    assert all(h.reason() == rt.FinishReason.Length for h in handles)
    # streaming channel delivers the same tokens and ends with a finished chunk
    ch = handles[1].stream()
    got, fin = [], False
    while True:
        c = ch.try_pop()
        if c is None:
            break
        got += c.token_ids
        fin = fin or c.finished
    assert got == outs[1] and fin
    m = eng.metrics()
    assert m.submitted == 4 and m.completed == 4 and m.admitted_mid_flight >= 1 and m.mixed_steps + m.prompt_steps >= 2
    assert handles[2].stats().ttft_s > 0
    # an over-long prompt is refused permanently, not retried
    h, _ = eng.submit(_req(1, n_prompt=100))
    with_err = h.get(10.0)
    assert with_err == [] and h.reason() == rt.FinishReason.Error and "TOO_LONG" in h.error()
    eng.shutdown()
    assert eng.status().resident == 0


def test_request_engine_cancel_and_refusals():
    cfg = rt.EngineConfig()
    cfg.max_batch_size, cfg.max_pending_requests = 1, 2
    opts = rt.SchedulingOptions()
    opts.min_request_priority = 1
    cfg.scheduling = opts
    eng = rt.RequestEngine(cfg, lambda: ScriptedSession(batch=1))
    h_low, why = eng.submit(_req(5, prio=0))
    assert h_low is None and "priority" in why
    long_req = _req(7, max_tokens=100000, prio=1)
    h1, _ = eng.submit(long_req)
    time.sleep(0.05)
    h2, _ = eng.submit(_req(9, prio=1))
    h3, _ = eng.submit(_req(11, prio=1))
    h4, why = eng.submit(_req(13, prio=1))
    assert h4 is None and why == "queue_full"
    h1.cancel()                           # consumer goes away: the seat frees at the next step boundary
    assert h2.get(10.0)[0] == 9 and h3.get(10.0)[0] == 11
    assert h1.reason() == rt.FinishReason.Cancelled
    m = eng.metrics()
    assert m.cancelled == 1 and m.refused == 2
    eng.shutdown()


def test_request_engine_session_failure_and_unavailable():
    made = []

    def factory():
        s = ScriptedSession(batch=2, fail_on_step=2 if len(made) < 2 else None)
        made.append(s)
        return s

    cfg = rt.EngineConfig()
    cfg.max_batch_size, cfg.max_consecutive_session_failures = 2, 2
    eng = rt.RequestEngine(cfg, factory)
    h, _ = eng.submit(_req(3, max_tokens=50))
    h.get(10.0)
    assert h.reason() == rt.FinishReason.Error and "injected" in h.error()
    assert eng.status().available and len(made) == 2          # session reopened after the first failure
    h2, _ = eng.submit(_req(4, max_tokens=50))
    h2.get(10.0)
    assert h2.reason() == rt.FinishReason.Error
    st = eng.status()
    assert not st.available and "engine_unavailable" in st.unavailable_reason
    h3, why = eng.submit(_req(5))
    assert h3 is None and "engine_unavailable" in why
    eng.shutdown()


def test_stream_channel_and_utf8():
    ch = rt.StreamChannel.create(True)
    ch.set_stream_interval(3)
    ch.push([1])
    ch.push([2])
    assert ch.try_pop() is None          # interval not reached
    ch.push([3])
    assert ch.try_pop().token_ids == [1, 2, 3]
    t = threading.Thread(target=lambda: (time.sleep(0.05), ch.push([4]), ch.finish(rt.FinishReason.EndId)))
    t.start()
    c = ch.wait_pop(2.0)
    t.join()
    assert c.token_ids == [4] and c.finished and c.reason == rt.FinishReason.EndId
    assert ch.metrics().generated_tokens == 4
    s = "héllo 世界".encode()
    assert rt.utf8_complete_prefix(s) == len(s)
    assert rt.utf8_complete_prefix(s[:-1]) == len(s) - 3 and rt.utf8_complete_prefix(s[:2]) == 1


def test_ragged_batch_and_sampler_and_config():
    pl = _planner(rt.IfbSchedulingMode.Mixed)
    plan = pl.plan([_res(0, 100, 64), _res(1, 20, 20, generated=2)])
    b = rt.build_ragged_batch(plan, [64, 21])
    assert b.q_start == [0, 36, 37] and b.positions[:3] == [64, 65, 66] and b.positions[-1] == 21
    assert b.logits_idx == [35, 36] and b.slot_ids == [0, 1] and b.max_seq_len == 100
    p = rt.RowSamplingParams()
    logits = np.array([0.1, 3.0, 2.9, -1.0], dtype=np.float32)
    assert rt.sample_row(logits, p, 0.7) == 1
    p.temperature, p.top_k = 1.0, 2
    picks = {rt.sample_row(logits, p, u) for u in np.linspace(0, 0.999, 50)}
    assert picks == {1, 2}
    p.top_k, p.top_p = 0, 0.3
    assert {rt.sample_row(logits, p, u) for u in np.linspace(0, 0.999, 20)} == {1}
    u1, u2 = rt.request_stable_uniform(42, 7, 3), rt.request_stable_uniform(42, 7, 3)
    assert u1 == u2 and 0 <= u1 < 1 and rt.request_stable_uniform(42, 8, 3) != u1
    c = rt.LLMEngineConfig.from_json(json.dumps({"model_type": "qwen3", "hidden_size": 4096, "num_attention_heads": 32,
                                                 "num_hidden_layers": 36, "decoding_strategies": ["vanilla", "eagle3"]}))
    assert c.head_dim == 128 and c.num_kv_heads == 32 and json.loads(c.to_json())["decoding_strategies"] == ["vanilla", "eagle3"]
    lm = rt.LoRAManager()
    a = rt.LoraAdapter()
    a.name, a.rank = "fr", 16
    lm.add(a)
    assert lm.activate("fr") and lm.active().rank == 16 and not lm.activate("nope")
    f = rt.DeviceFailureState()
    f.record("first")
    f.record("second")
    assert f.failed() and f.reason() == "first"
    assert json.loads(rt.json_roundtrip('{"a":[1,2.5,"x\\u00e9\\ud83d\\ude00"],"b":{"c":null,"d":true}}'))["a"][2] == "xé😀"


TEXTS = ["Hello, world!", "  leading and   multiple   spaces ", "it's we're I'll they've don't", "line1\nline2\r\n\r\nline3",
         "numbers 12345 and 3.14159", "mixed: naïve café — “quotes” … ok?", "中文字符和English混合", "def f(x):\n    return x**2  # sq",
         "tabs\tand\ttabs", "trailing space ", "a", ""]


@pytest.fixture(scope="module")
def hf_tok(tmp_path_factory):
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE())
    pat = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pat), behavior="isolated"),
                                                 pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=600, special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    corpus = TEXTS * 3 + ["the quick brown fox jumps over the lazy dog " * 5, "hello hello world world 你好 你好"]
    tok.train_from_iterator(corpus, trainer)
    d = tmp_path_factory.mktemp("tok")
    tok.save(str(d / "tokenizer.json"))
    (d / "tokenizer_config.json").write_text(json.dumps({"eos_token": "<|im_end|>", "chat_template": "{% for m in messages %}<|im_start|>..."}))
    return tok, str(d)


def test_tokenizer_matches_hf(hf_tok):
    tok, d = hf_tok
    mine = rt.Tokenizer.load_from_hf(d)
    assert mine.vocab_size == tok.get_vocab_size() and mine.eos_id == tok.token_to_id("<|im_end|>")
    for text in TEXTS + ["<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"]:
        want = tok.encode(text).ids
        got = mine.encode(text)
        assert got == want, (text, got, want)
        assert mine.decode(got, False).decode() == text
    assert mine.is_special(mine.eos_id) and mine.decode([mine.eos_id]).decode() == ""


def test_tokenizer_unicode_classes_match_hf(hf_tok):
    """Pre-tokenisation splits on exact Unicode letter / number / white-space classes: scripts, numerals and marks that a
    hand-written range list gets wrong must split as the Hugging Face regex engine splits them."""
    tok, d = hf_tok
    mine = rt.Tokenizer.load_from_hf(d)
    texts = ["Ⅻ世紀 x²+y³=½ ٣٤٥ ১২৩ ௧௨", "e\u0301cole na\u0308ive", "ไทย123ไทย ᠮᠣᠩᠭᠣᠯ", "αβγ·δ 한국어—テスト　全角", "a\u2028b\u00a0c\u1680d\u001ce",
             "🙂 emoji👍🏽mix", "ℵ₀ ∑ᵢxᵢ ℃ №5 ㈱ ①②③ 𝒜𝔅 𐍈", "ǅ ʰ ʻokina ˈstress ՙ ֊", "x\u200by\ufeffz \u0600\u06dd"]
    for text in texts:
        want = tok.encode(text).ids
        got = mine.encode(text)
        assert got == want, (text, got, want)
        assert mine.decode(got, False).decode() == text


def test_chat_template_families(hf_tok):
    _, d = hf_tok
    ct = rt.ChatTemplate.load(d)
    msgs = [rt.ChatMessage("system", "be brief"), rt.ChatMessage("user", "hi")]
    assert ct.apply(msgs) == "<|im_start|>system\nbe brief<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    l3 = rt.ChatTemplate.from_template_text("{{ '<|start_header_id|>' }}", "<|begin_of_text|>")
    assert l3.apply([rt.ChatMessage("user", "hi")]).startswith("<|begin_of_text|><|start_header_id|>user<|end_header_id|>\n\nhi<|eot_id|>")
    l2 = rt.ChatTemplate.from_template_text("[INST] {{ x }} [/INST]", "<s>")
    assert l2.apply(msgs) == "<s>[INST] <<SYS>>\nbe brief\n<</SYS>>\n\nhi [/INST]"


def test_kernel_library_load_failure_is_loud(monkeypatch):
    """The fault-injection switch makes the kernel library fail to load; nothing falls back silently."""
    from tensorrt_edge_llm_b200.ops import cuda as cu
    monkeypatch.setattr(cu, "_lib", None)
    monkeypatch.setenv("TELB_TEST_FAIL_KERNEL_LIBRARY", "1")
    with pytest.raises(RuntimeError, match="failed to load"):
        cu.lib()
    monkeypatch.delenv("TELB_TEST_FAIL_KERNEL_LIBRARY")
    assert cu.lib() is not None


def test_prefix_cache_eviction_planner_and_chain_order():
    """Eviction is planned read-only first: only pages whose last reference is the cache's count, shared pages are passed over,
    and a chain's later pages go before the pages every continuation of the prefix depends on."""
    t = rt.KVPageTable(num_pages=12, page_size=4, max_seats=3, max_pages_per_seq=6)
    cache = rt.PrefixCache(t.allocator(), 4, 16)
    a = list(range(100, 117))                       # 17 tokens: 4 full pages
    t.reserve(0, 17)
    assert cache.insert(a, 16, t.pages(0)) == 4
    pages_a = list(t.pages(0))
    t.free_seat(0)                                  # the cache now holds the only reference on 4 pages
    b = a[:8] + list(range(200, 209))               # shares the first two pages, then diverges
    m = cache.lookup(b)
    assert m.tokens == 8 and m.pages == pages_a[:2]
    t.adopt_prefix(1, m.pages, m.tokens)            # a resident sequence shares pages 0 and 1
    free0 = t.free_pages
    # read-only plan: pages 2 and 3 of chain a (its leaves) are reclaimable, the shared ones are passed over
    plan = cache.plan_eviction(3)
    assert plan.reclaimable_pages == 2 and not plan.satisfied and plan.pinned_skipped == 2 and len(plan.victims) == 2
    assert cache.records == 4 and t.free_pages == free0                    # nothing changed
    plan1 = cache.plan_eviction(1)
    assert plan1.satisfied and len(plan1.victims) == 1
    assert cache.evict_plan(plan1) == 1 and t.free_pages == free0 + 1 and cache.records == 3
    # the victim was the chain's last page: the first three pages still match
    assert cache.lookup(a).tokens == 12
    # evict(n) returns pages actually freed and never drops records that would free nothing
    assert cache.evict(5) == 1 and cache.records == 2 and t.free_pages == free0 + 2
    assert cache.evict(5) == 0 and cache.records == 2
    assert cache.lookup(a).tokens == 8                                     # the shared root pages are still indexed
    t.free_seat(1)
    assert cache.evict(5) == 2 and cache.records == 0 and t.free_pages == 12
    # a stale plan is harmless: its victims are gone
    assert cache.evict_plan(plan) == 0
    # the record limit drops the oldest records whatever their state
    small = rt.PrefixCache(t.allocator(), 4, 2)
    t.reserve(2, 13)
    assert small.insert(list(range(13)), 12, t.pages(2)) == 3 and small.records == 2
    assert small.drop_records(5) == 2 and small.records == 0


def test_engine_config_from_a_prepared_models_runtime_config():
    """The native config reads what `trtedge build` records: model geometry, quantisation, per-layer types, recurrent and draft
    sections, deployment limits; its derived sizes match the Python cache manager's, and validation names the first problem."""
    import dataclasses
    from tensorrt_edge_llm_b200.checkpoint.artifacts import runtime_config_dict
    from tensorrt_edge_llm_b200.config import GdnConfig, MambaConfig, QuantConfig, hybrid_nemotron_config, qwen3_8b_config
    from tensorrt_edge_llm_b200.runtime.kv_cache import KVCacheManager
    dense = qwen3_8b_config(dtype="float16", quant=QuantConfig(quant_type="nvfp4", group_size=16))
    text = json.dumps(runtime_config_dict(dense, 64, 1024, 1216, 1), default=str)
    c = rt.LLMEngineConfig.from_runtime_config(text)
    assert (c.model_type, c.num_layers, c.num_heads, c.num_kv_heads, c.head_dim, c.vocab_size) == ("qwen3", 36, 32, 8, 128, 151936)
    assert (c.quantization, c.quant_group_size, c.max_batch_size, c.max_input_len, c.max_kv_cache_capacity, c.kv_page_size) == ("nvfp4", 16, 64, 1024, 1216, 64)
    assert c.has_qk_norm and c.rotary_dim == 128 and c.rope_theta == 1e6 and not c.is_hybrid() and not c.is_moe() and c.validate() == ""
    assert c.num_attention_layers() == 36 and c.kv_bytes_per_token() == 2 * 36 * 8 * 128 * 2
    kv = KVCacheManager(qwen3_8b_config(dtype="float16", num_hidden_layers=2), num_pages=8, page_size=64, max_seats=1, max_pages_per_seq=4)
    assert kv.pool.element_size() * kv.pool[0, 0].numel() // 64 * 36 == c.kv_bytes_per_token()
    assert c.kv_pool_bytes() == c.kv_bytes_per_token() * 64 * (19 * 64 + 1)
    hyb = hybrid_nemotron_config(num_hidden_layers=8, vocab_size=500, hidden_size=64, intermediate_size=128, num_attention_heads=4,
                                 num_key_value_heads=2, head_dim=16, dtype="bfloat16", max_position_embeddings=512,
                                 mamba=MambaConfig(num_heads=4, head_dim=8, d_state=16, n_groups=2, conv_kernel=4),
                                 gdn=GdnConfig(num_k_heads=2, num_v_heads=4, head_k_dim=8, head_v_dim=8, conv_kernel=4))
    h = rt.LLMEngineConfig.from_runtime_config(json.dumps(runtime_config_dict(hyb, 2, 64, 128, 1), default=str))
    assert h.is_hybrid() and h.num_recurrent_layers() == sum(t in ("mamba", "gdn") for t in hyb.layer_types)
    assert h.num_attention_layers() == sum(t == "attention" for t in hyb.layer_types) and h.mamba_d_state == 16 and h.gdn_num_v_heads == 4
    from tensorrt_edge_llm_b200.models.nemotron_h import RecurrentState
    st = RecurrentState(hyb, 1, "cpu", torch.bfloat16)
    assert h.recurrent_state_bytes_per_seat() == sum(t.numel() * t.element_size() for t in st.pools())
    # validation
    bad = rt.LLMEngineConfig.from_runtime_config(text)
    bad.num_kv_heads = 5
    assert "multiple" in bad.validate()
    bad = rt.LLMEngineConfig.from_runtime_config(text)
    bad.max_kv_cache_capacity = 100
    assert "max_kv_cache_capacity" in bad.validate()
    bad = rt.LLMEngineConfig.from_runtime_config(text)
    bad.layer_types = ["attention"] * 3
    assert "layer_types" in bad.validate()
    draft = dataclasses.replace(dense, draft_type="dflash", dflash_block_size=8, dflash_version=2, dflash_projector_type="lilicorr")
    d = rt.LLMEngineConfig.from_runtime_config(json.dumps(runtime_config_dict(draft, 1, 64, 128, 1), default=str))
    assert (d.draft_type, d.dflash_block_size, d.dflash_version, d.dflash_projector_type) == ("dflash", 8, 2, "lilicorr")
