// Hugging Face `tokenizer.json` BPE tokenizer: byte-level (GPT-2 / Qwen / Llama-3 style, with the
// regex pre-tokeniser implemented as a hand-written scanner) and metaspace + byte-fallback
// (Llama-2 / Mistral style).  encode / decode / id_to_piece / load_from_hf.
//
// Counterpart of cpp/tokenizer/tokenizer.{h,cpp} in the reference (which carries generated Unicode
// tables, cpp/tokenizer/unicodeData.cpp).  The letter, number and white-space classes of the
// pre-tokeniser come from exact range tables (unicode_tables.inc, written by gen_unicode_tables.py
// from Python's unicodedata), searched by bisection.
#pragma once

#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

namespace telb {

class Tokenizer {
  public:
    // Reads <dir>/tokenizer.json (and tokenizer_config.json for bos/eos names when present).
    static Tokenizer load_from_hf(const std::string& dir_or_file);
    static Tokenizer from_json_text(const std::string& tokenizer_json, const std::string& config_json = "");

    std::vector<int32_t> encode(const std::string& text, bool add_special_tokens = false) const;
    std::string decode(const std::vector<int32_t>& ids, bool skip_special_tokens = true) const;
    // Raw bytes of one token (may be an incomplete UTF-8 sequence; stream through utf8_complete_prefix).
    std::string id_to_bytes(int32_t id) const;
    const std::string& id_to_piece(int32_t id) const;
    int32_t piece_to_id(const std::string& piece) const;      // -1 when unknown
    int vocab_size() const { return static_cast<int>(id_to_piece_.size()); }
    int32_t bos_id() const { return bos_id_; }
    int32_t eos_id() const { return eos_id_; }
    bool is_special(int32_t id) const { return id >= 0 && id < static_cast<int>(special_.size()) && special_[id]; }

  private:
    void bpe(const std::string& word, std::vector<int32_t>& out) const;
    void encode_plain(const std::string& text, std::vector<int32_t>& out) const;
    std::vector<std::string> pre_tokenize(const std::string& text) const;

    bool byte_level_ = true;            // false: metaspace + byte fallback
    bool add_prefix_space_ = false;
    bool prepend_metaspace_ = true;
    std::unordered_map<std::string, int32_t> vocab_;
    std::vector<std::string> id_to_piece_;
    std::unordered_map<std::string, int32_t> merge_rank_;       // "left right" -> rank
    std::vector<std::pair<std::string, int32_t>> added_;        // literal → id, longest first
    std::vector<uint8_t> special_;
    int32_t bos_id_ = -1, eos_id_ = -1, unk_id_ = -1;
    bool add_bos_ = false;
    std::string byte_to_uni_[256];
    std::unordered_map<std::string, uint8_t> uni_to_byte_;
    int32_t byte_fallback_[256];
};

// Chat prompt construction.  The template string from tokenizer_config.json is recognised by
// family (ChatML / Llama-3 / Llama-2-INST / plain) and rendered natively; arbitrary Jinja is the
// Python layer's job (tensorrt_edge_llm_b200.chat_template).
struct ChatMessage {
    std::string role, content;
};

class ChatTemplate {
  public:
    enum class Family { kChatML, kLlama3, kLlama2, kPlain };
    static ChatTemplate load(const std::string& model_dir);
    static ChatTemplate from_template_text(const std::string& jinja_text, const std::string& bos = "");
    std::string apply(const std::vector<ChatMessage>& messages, bool add_generation_prompt = true,
                      bool enable_thinking = true) const;
    Family family() const { return family_; }
    const std::string& source() const { return source_; }

  private:
    Family family_ = Family::kChatML;
    std::string source_, bos_;
    std::string default_system_;
};

}  // namespace telb
