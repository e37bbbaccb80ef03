"""The native façade (``csrc/runtime/inference_runtime.cpp``) with a scripted session: chat rendering and tokenisation,
in-flight batching of a request batch, incremental detokenisation, textual stop sequences, refusals, streaming callbacks."""
import json

import pytest

from tensorrt_edge_llm_b200.runtime import native as rt


@pytest.fixture(scope="module")
def tok_dir(tmp_path_factory):
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE())
    pat = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"
    tok.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pat), behavior="isolated"),
                                                 pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=400, special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(["the quick brown fox jumps over the lazy dog " * 4, "hello world STOP here 你好"] * 3, trainer)
    d = tmp_path_factory.mktemp("tokrt")
    tok.save(str(d / "tokenizer.json"))
    (d / "tokenizer_config.json").write_text(json.dumps({"eos_token": "<|im_end|>", "chat_template": "{% for m in messages %}<|im_start|>..."}))
    return str(d)


class ReplaySession(rt.RuntimeSession):
    """Generates, for every request, the token list ``scripts[first prompt token]`` (cycled), one token per step."""

    def __init__(self, scripts, batch=2):
        super().__init__()
        self.scripts, self.batch = scripts, batch
        self.free, self.seqs, self.prompts, self.max_rows = list(range(batch)), {}, [], 0

    def capabilities(self):
        c = rt.SessionCapabilities()
        c.compact, c.max_batch_size, c.max_input_length, c.kv_page_size, c.max_kv_tokens = True, self.batch, 256, 16, 1024
        return c

    def admit(self, request_id, req):
        r = rt.AdmissionResult()
        if not self.free:
            r.admitted, r.retry_later, r.reason = False, True, "no seat"
            return r
        r.admitted, r.slot = True, self.free.pop(0)
        self.seqs[r.slot] = (list(req.prompt_ids), 0)
        self.prompts.append(list(req.prompt_ids))
        return r

    def execute(self, plan):
        out, deltas = rt.StepResult(), []
        self.max_rows = max(self.max_rows, len(plan.seqs))
        for s in plan.seqs:
            prompt, gen = self.seqs[s.slot]
            if s.kind == rt.WorkKind.Context and not s.last_chunk:
                continue
            script = self.scripts[prompt[-1]] if prompt[-1] in self.scripts else self.scripts["default"]
            d = rt.TokenDelta()
            d.slot, d.tokens = s.slot, [script[gen % len(script)]]
            self.seqs[s.slot] = (prompt, gen + 1)
            deltas.append(d)
        out.deltas = deltas
        return out

    def release(self, slot):
        self.seqs.pop(slot, None)
        self.free.append(slot)


def _runtime(tok_dir, scripts, batch=2, hook=None):
    tok = rt.Tokenizer.load_from_hf(tok_dir)
    tpl = rt.ChatTemplate.load(tok_dir)
    sessions = []

    def factory():
        s = ReplaySession(scripts, batch)
        sessions.append(s)
        return s

    cfg = rt.EngineConfig()
    cfg.max_batch_size = batch
    return rt.LLMInferenceRuntime(cfg, factory, tok, tpl, False, hook), tok, tpl, sessions


def _entry(prompt=None, messages=None, ids=None):
    e = rt.GenerationEntry()
    if prompt is not None:
        e.prompt = prompt
    if messages is not None:
        ms = []
        for role, content in messages:
            m = rt.ChatMessage()
            m.role, m.content = role, content
            ms.append(m)
        e.messages = ms
    if ids is not None:
        e.prompt_ids = ids
    return e


def test_batch_of_chats_and_prompts(tok_dir):
    tok0 = rt.Tokenizer.load_from_hf(tok_dir)
    reply = tok0.encode("the quick brown fox")
    runtime, tok, tpl, sessions = _runtime(tok_dir, {"default": reply})
    req = rt.LLMGenerationRequest()
    req.requests = [_entry(messages=[("user", "hello world")]), _entry(prompt="the lazy dog"), _entry(ids=[5, 6, 7])]
    req.max_generate_length = len(reply)
    seen = {}
    resp = runtime.handle_request(req, lambda i, toks, text, fin: seen.setdefault(i, []).append((list(toks), text, fin)))
    assert resp.output_texts == ["the quick brown fox"] * 3 and resp.output_ids == [reply] * 3
    assert all(r == rt.FinishReason.Length for r in resp.finish_reasons) and resp.errors == ["", "", ""]
    assert [s.prompt_tokens for s in resp.stats][2] == 3 and all(s.generated_tokens == len(reply) for s in resp.stats)
    # the chat entry went through the template, the plain prompt did not
    msg = rt.ChatMessage()
    msg.role, msg.content = "user", "hello world"
    assert sessions[0].prompts[0] == tok.encode(tpl.apply([msg], True, True)) and sessions[0].prompts[1] == tok.encode("the lazy dog", True)
    assert runtime.count_prompt_tokens(req, req.requests[2]) == 3
    # three requests, two seats: batched in flight, the third admitted when a seat frees up
    assert sessions[0].max_rows == 2 and runtime.metrics().completed == 3
    # streamed pieces concatenate to the text and end with a finished call
    for i in range(3):
        assert "".join(t for _, t, _ in seen[i]) == "the quick brown fox" and seen[i][-1][2]
        assert [x for toks, _, _ in seen[i] for x in toks] == reply
    assert runtime.supports_seated_admission() and runtime.supports_stepped_execution() and not runtime.has_draft_model()
    assert runtime.unavailable_reason() == ""
    runtime.shutdown()


def test_textual_stop_sequence_and_utf8_boundaries(tok_dir):
    tok0 = rt.Tokenizer.load_from_hf(tok_dir)
    text = "hello 你好 world STOP here the quick"
    script = tok0.encode(text)
    runtime, tok, _, _ = _runtime(tok_dir, {"default": script}, batch=1)
    req = rt.LLMGenerationRequest()
    req.requests = [_entry(ids=[9])]
    req.max_generate_length, req.stop = len(script), ["STOP", "never"]
    pieces = []
    resp = runtime.handle_request(req, lambda i, toks, t, fin: pieces.append(t))
    assert resp.output_texts == ["hello 你好 world "] and resp.finish_reasons == [rt.FinishReason.StopWords] and resp.errors == [""]
    assert "".join(pieces) == "hello 你好 world " and all("�" not in p for p in pieces)     # multi-byte characters never split
    assert len(resp.output_ids[0]) < len(script)
    # without the stop sequence the whole script comes back
    req.stop = []
    assert runtime.handle_request(req).output_texts == [text]
    runtime.shutdown()


def test_malformed_batches_refusals_and_hooks(tok_dir):
    calls = []
    runtime, tok, _, _ = _runtime(tok_dir, {"default": [7]}, hook=lambda: (calls.append(1), True)[1])
    with pytest.raises(RuntimeError, match="empty request batch"):
        runtime.handle_request(rt.LLMGenerationRequest())
    req = rt.LLMGenerationRequest()
    req.requests, req.max_generate_length = [_entry(ids=[1])], 0
    with pytest.raises(RuntimeError, match="max_generate_length"):
        runtime.handle_request(req)
    req.max_generate_length, req.stop = 2, [""]
    with pytest.raises(RuntimeError, match="empty stop"):
        runtime.handle_request(req)
    # an entry with nothing in it fails alone; its neighbours still run
    req.stop, req.requests = [], [_entry(prompt=""), _entry(ids=[3, 4])]
    resp = runtime.handle_request(req)
    assert resp.errors[0] == "empty prompt" and resp.finish_reasons[0] == rt.FinishReason.Error and resp.output_ids[1] == [7, 7]
    # the capture hook runs only while the engine is idle
    assert runtime.capture_decoding_cuda_graph() and calls == [1]
    # seated admission hands back a handle; stepped execution a session of one's own
    g = rt.GenerationRequest()
    g.prompt_ids, g.max_tokens = [2, 2], 3
    handle, why = runtime.submit(g)
    assert why == "" and handle.get(10.0) == [7, 7, 7]
    assert isinstance(runtime.open_session(), rt.RuntimeSession)
    runtime.shutdown()


def test_llm_serves_request_batches_through_the_native_facade(tok_dir):
    """A model behind the façade: ``LLM`` with a native tokenizer starts its request engine inside the native runtime object,
    and a request batch decodes to the same tokens as the static path."""
    from tensorrt_edge_llm_b200.config import tiny_llama_config
    from tensorrt_edge_llm_b200.runtime.llm import LLM
    from tensorrt_edge_llm_b200.runtime.runner import SamplingParams
    tok = rt.Tokenizer.load_from_hf(tok_dir)
    cfg = tiny_llama_config(num_hidden_layers=2, vocab_size=512, dtype="float32")
    static = LLM(cfg, device="cpu", max_batch_size=4, max_input_len=128, max_kv_cache_capacity=192, random_init_seed=3)
    llm = LLM(cfg, device="cpu", max_batch_size=2, max_input_len=128, max_kv_cache_capacity=192, random_init_seed=3, tokenizer=tok,
              enable_in_flight_batching=True)
    assert isinstance(llm.native_runtime, rt.LLMInferenceRuntime) and llm.engine is llm.native_runtime
    req = rt.LLMGenerationRequest()
    req.requests = [_entry(prompt="the quick brown fox"), _entry(prompt="hello world"), _entry(ids=[11, 12, 13, 14])]
    req.max_generate_length, req.ignore_eos = 6, True
    resp = llm.native_runtime.handle_request(req)
    prompts = [tok.encode("the quick brown fox", True), tok.encode("hello world", True), [11, 12, 13, 14]]
    want = static.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
    assert resp.output_ids == [list(w.token_ids) if hasattr(w, "token_ids") else list(w) for w in want]
    assert resp.output_texts == [tok.decode(ids, True).decode("utf-8", "replace") for ids in resp.output_ids]
    # the ordinary submit path still works on the same object
    assert llm.submit(prompts[1], SamplingParams(max_tokens=3, ignore_eos=True)).get(30.0) == resp.output_ids[1][:3]
    llm.close(); static.close()
