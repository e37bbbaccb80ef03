#include "tokenizer.h"

#include <algorithm>
#include <climits>
#include <fstream>
#include <sstream>
#include <stdexcept>

#include "json.h"

namespace telb {

// ---- UTF-8 helpers ------------------------------------------------------------------------------
static uint32_t next_cp(const std::string& s, size_t& i) {
    const unsigned char c = static_cast<unsigned char>(s[i]);
    uint32_t cp = c;
    int extra = 0;
    if (c >= 0xF0) { cp = c & 0x07; extra = 3; }
    else if (c >= 0xE0) { cp = c & 0x0F; extra = 2; }
    else if (c >= 0xC0) { cp = c & 0x1F; extra = 1; }
    ++i;
    for (int k = 0; k < extra && i < s.size(); ++k, ++i) cp = (cp << 6) | (static_cast<unsigned char>(s[i]) & 0x3F);
    return cp;
}
static void put_cp(std::string& o, uint32_t cp) {
    if (cp < 0x80) o += static_cast<char>(cp);
    else if (cp < 0x800) { o += static_cast<char>(0xC0 | (cp >> 6)); o += static_cast<char>(0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) {
        o += static_cast<char>(0xE0 | (cp >> 12)); o += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
        o += static_cast<char>(0x80 | (cp & 0x3F));
    } else {
        o += static_cast<char>(0xF0 | (cp >> 18)); o += static_cast<char>(0x80 | ((cp >> 12) & 0x3F));
        o += static_cast<char>(0x80 | ((cp >> 6) & 0x3F)); o += static_cast<char>(0x80 | (cp & 0x3F));
    }
}

// ---- Unicode classes of the pre-tokenisation patterns (\p{L}, \p{N}, \s): exact range tables ------------------------
#include "unicode_tables.inc"

static bool in_ranges(const uint32_t (*r)[2], int n, uint32_t c) {
    int lo = 0, hi = n - 1;
    while (lo <= hi) {
        const int mid = (lo + hi) >> 1;
        if (c < r[mid][0]) hi = mid - 1;
        else if (c > r[mid][1]) lo = mid + 1;
        else return true;
    }
    return false;
}
static bool is_space_cp(uint32_t c) {
    if (c < 0x80) return c == ' ' || (c >= 9 && c <= 13);
    return in_ranges(kUnicodeWhiteSpace, kUnicodeWhiteSpace_count, c);
}
static bool is_digit_cp(uint32_t c) {
    if (c < 0x80) return c >= '0' && c <= '9';
    return in_ranges(kUnicodeNumber, kUnicodeNumber_count, c);
}
static bool is_letter_cp(uint32_t c) {
    if (c < 0x80) return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z');
    return in_ranges(kUnicodeLetter, kUnicodeLetter_count, c);
}

// ---- loading ------------------------------------------------------------------------------------
static std::string read_file(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot open " + path);
    std::ostringstream ss;
    ss << f.rdbuf();
    return ss.str();
}

Tokenizer Tokenizer::load_from_hf(const std::string& dir_or_file) {
    std::string path = dir_or_file, cfg;
    if (path.size() < 5 || path.substr(path.size() - 5) != ".json") {
        const std::string dir = path;
        path = dir + "/tokenizer.json";
        std::ifstream c(dir + "/tokenizer_config.json");
        if (c) {
            std::ostringstream ss;
            ss << c.rdbuf();
            cfg = ss.str();
        }
    }
    return from_json_text(read_file(path), cfg);
}

Tokenizer Tokenizer::from_json_text(const std::string& text, const std::string& config_json) {
    Tokenizer t;
    const Json root = Json::parse(text);
    const Json& model = root["model"];
    if (model["type"].as_string() != "BPE" && !model["type"].is_null())
        throw std::runtime_error("tokenizer model type '" + model["type"].as_string() + "' is not supported (BPE only)");
    // GPT-2 byte <-> unicode table
    {
        std::vector<int> bs;
        for (int b = '!'; b <= '~'; ++b) bs.push_back(b);
        for (int b = 0xA1; b <= 0xAC; ++b) bs.push_back(b);
        for (int b = 0xAE; b <= 0xFF; ++b) bs.push_back(b);
        std::vector<int> cs = bs;
        int n = 0;
        for (int b = 0; b < 256; ++b)
            if (std::find(bs.begin(), bs.end(), b) == bs.end()) { bs.push_back(b); cs.push_back(256 + n++); }
        for (size_t i = 0; i < bs.size(); ++i) {
            std::string u;
            put_cp(u, static_cast<uint32_t>(cs[i]));
            t.byte_to_uni_[bs[i]] = u;
            t.uni_to_byte_[u] = static_cast<uint8_t>(bs[i]);
        }
    }
    int max_id = -1;
    for (const auto& kv : model["vocab"].members()) {
        const int32_t id = static_cast<int32_t>(kv.second.as_int());
        t.vocab_[kv.first] = id;
        max_id = std::max(max_id, id);
    }
    for (const auto& a : root["added_tokens"].items()) max_id = std::max<int>(max_id, static_cast<int>(a["id"].as_int()));
    t.id_to_piece_.assign(max_id + 1, std::string());
    t.special_.assign(max_id + 1, 0);
    for (const auto& kv : t.vocab_) t.id_to_piece_[kv.second] = kv.first;
    int rank = 0;
    for (const auto& m : model["merges"].items()) {
        std::string key;
        if (m.is_string()) key = m.as_string();
        else if (m.is_array() && m.size() == 2) key = m[0].as_string() + " " + m[1].as_string();
        t.merge_rank_[key] = rank++;
    }
    for (const auto& a : root["added_tokens"].items()) {
        const int32_t id = static_cast<int32_t>(a["id"].as_int());
        const std::string& content = a["content"].as_string();
        t.added_.emplace_back(content, id);
        t.id_to_piece_[id] = content;
        t.vocab_[content] = id;
        if (a["special"].as_bool(false)) t.special_[id] = 1;
    }
    std::sort(t.added_.begin(), t.added_.end(), [](const auto& a, const auto& b) { return a.first.size() > b.first.size(); });
    t.byte_level_ = !model["byte_fallback"].as_bool(false);
    if (!t.byte_level_) {
        for (int b = 0; b < 256; ++b) {
            char buf[8];
            snprintf(buf, sizeof(buf), "<0x%02X>", b);
            auto it = t.vocab_.find(buf);
            t.byte_fallback_[b] = it == t.vocab_.end() ? -1 : it->second;
        }
        const Json& norm = root["normalizer"];
        t.prepend_metaspace_ = norm.dump().find("Prepend") != std::string::npos || root["pre_tokenizer"].dump().find("Metaspace") != std::string::npos;
    } else {
        t.add_prefix_space_ = root["pre_tokenizer"].dump().find("\"add_prefix_space\":true") != std::string::npos;
    }
    const std::string unk = model["unk_token"].as_string();
    if (!unk.empty()) t.unk_id_ = t.piece_to_id(unk);
    if (!config_json.empty()) {
        const Json cfg = Json::parse(config_json);
        auto tok_name = [&](const char* key) -> std::string {
            const Json& v = cfg[key];
            if (v.is_string()) return v.as_string();
            if (v.is_object()) return v["content"].as_string();
            return "";
        };
        const std::string bos = tok_name("bos_token"), eos = tok_name("eos_token");
        if (!bos.empty()) t.bos_id_ = t.piece_to_id(bos);
        if (!eos.empty()) t.eos_id_ = t.piece_to_id(eos);
        t.add_bos_ = cfg["add_bos_token"].as_bool(false);
    }
    if (t.eos_id_ < 0)
        for (const char* cand : {"<|im_end|>", "<|endoftext|>", "</s>", "<|eot_id|>", "<|end_of_text|>"}) {
            const int32_t id = t.piece_to_id(cand);
            if (id >= 0) { t.eos_id_ = id; break; }
        }
    if (t.bos_id_ < 0)
        for (const char* cand : {"<s>", "<|begin_of_text|>"}) {
            const int32_t id = t.piece_to_id(cand);
            if (id >= 0) { t.bos_id_ = id; break; }
        }
    return t;
}

int32_t Tokenizer::piece_to_id(const std::string& piece) const {
    auto it = vocab_.find(piece);
    return it == vocab_.end() ? -1 : it->second;
}

const std::string& Tokenizer::id_to_piece(int32_t id) const {
    static const std::string empty;
    return (id >= 0 && id < static_cast<int>(id_to_piece_.size())) ? id_to_piece_[id] : empty;
}

// ---- pre-tokenisation (scanner equivalent of the GPT-4 / Qwen2 split pattern) -----------------------
//   (?i:'s|'t|'re|'ve|'m|'ll|'d) | [^\r\n\p{L}\p{N}]?\p{L}+ | \p{N} | ?[^\s\p{L}\p{N}]+[\r\n]* | \s*[\r\n]+ | \s+(?!\S) | \s+
std::vector<std::string> Tokenizer::pre_tokenize(const std::string& text) const {
    std::vector<uint32_t> cps;
    std::vector<size_t> off;
    for (size_t i = 0; i < text.size();) {
        off.push_back(i);
        cps.push_back(next_cp(text, i));
    }
    off.push_back(text.size());
    const size_t n = cps.size();
    std::vector<std::string> out;
    auto emit = [&](size_t a, size_t b) { out.push_back(text.substr(off[a], off[b] - off[a])); };
    auto lower = [](uint32_t c) { return (c >= 'A' && c <= 'Z') ? c + 32 : c; };
    size_t i = 0;
    while (i < n) {
        const uint32_t c = cps[i];
        // contractions
        if (c == '\'' && i + 1 < n) {
            const uint32_t a = lower(cps[i + 1]);
            const uint32_t b = i + 2 < n ? lower(cps[i + 2]) : 0;
            if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) { emit(i, i + 3); i += 3; continue; }
            if (a == 's' || a == 't' || a == 'm' || a == 'd') { emit(i, i + 2); i += 2; continue; }
        }
        // [^\r\n\p{L}\p{N}]?\p{L}+
        if (is_letter_cp(c) || (c != '\r' && c != '\n' && !is_digit_cp(c) && i + 1 < n && is_letter_cp(cps[i + 1]))) {
            size_t j = is_letter_cp(c) ? i : i + 1;
            while (j < n && is_letter_cp(cps[j])) ++j;
            emit(i, j);
            i = j;
            continue;
        }
        if (is_digit_cp(c)) { emit(i, i + 1); ++i; continue; }
        //  ?[^\s\p{L}\p{N}]+[\r\n]*
        {
            size_t j = i;
            if (c == ' ' && i + 1 < n) ++j;
            size_t k = j;
            while (k < n && !is_space_cp(cps[k]) && !is_letter_cp(cps[k]) && !is_digit_cp(cps[k])) ++k;
            if (k > j) {
                while (k < n && (cps[k] == '\r' || cps[k] == '\n')) ++k;
                emit(i, k);
                i = k;
                continue;
            }
        }
        // whitespace runs
        if (is_space_cp(c)) {
            size_t j = i;
            while (j < n && is_space_cp(cps[j])) ++j;
            // \s*[\r\n]+ : up to and including the last newline of the run
            size_t last_nl = SIZE_MAX;
            for (size_t k = i; k < j; ++k)
                if (cps[k] == '\r' || cps[k] == '\n') last_nl = k;
            if (last_nl != SIZE_MAX) { emit(i, last_nl + 1); i = last_nl + 1; continue; }
            // \s+(?!\S): leave the last space to glue to the next word, unless the run ends the text
            if (j < n && j - i > 1) { emit(i, j - 1); i = j - 1; continue; }
            if (j < n && j - i == 1) {
                // a single space followed by a non-space: it belongs to the next token (handled above for letters / symbols);
                // reaching here means the next char is a digit
                emit(i, j);
                i = j;
                continue;
            }
            emit(i, j);
            i = j;
            continue;
        }
        emit(i, i + 1);
        ++i;
    }
    return out;
}

void Tokenizer::bpe(const std::string& word, std::vector<int32_t>& out) const {
    // symbols = UTF-8 characters of the (byte-mapped) word
    std::vector<std::string> sym;
    for (size_t i = 0; i < word.size();) {
        const size_t s = i;
        next_cp(word, i);
        sym.push_back(word.substr(s, i - s));
    }
    while (sym.size() > 1) {
        int best = INT_MAX;
        size_t at = 0;
        for (size_t i = 0; i + 1 < sym.size(); ++i) {
            auto it = merge_rank_.find(sym[i] + " " + sym[i + 1]);
            if (it != merge_rank_.end() && it->second < best) { best = it->second; at = i; }
        }
        if (best == INT_MAX) break;
        sym[at] += sym[at + 1];
        sym.erase(sym.begin() + at + 1);
    }
    for (const auto& s : sym) {
        auto it = vocab_.find(s);
        if (it != vocab_.end()) { out.push_back(it->second); continue; }
        if (!byte_level_) {
            bool ok = true;
            for (unsigned char b : s) ok = ok && byte_fallback_[b] >= 0;
            if (ok) { for (unsigned char b : s) out.push_back(byte_fallback_[b]); continue; }
        }
        if (unk_id_ >= 0) out.push_back(unk_id_);
    }
}

void Tokenizer::encode_plain(const std::string& text, std::vector<int32_t>& out) const {
    if (text.empty()) return;
    if (byte_level_) {
        const std::string t = (add_prefix_space_ && text[0] != ' ') ? " " + text : text;
        for (const std::string& piece : pre_tokenize(t)) {
            std::string mapped;
            for (unsigned char b : piece) mapped += byte_to_uni_[b];
            auto it = vocab_.find(mapped);
            if (it != vocab_.end()) out.push_back(it->second);
            else bpe(mapped, out);
        }
    } else {
        std::string t;
        if (prepend_metaspace_) t = "\xE2\x96\x81";
        for (char c : text) {
            if (c == ' ') t += "\xE2\x96\x81";
            else t += c;
        }
        bpe(t, out);
    }
}

std::vector<int32_t> Tokenizer::encode(const std::string& text, bool add_special_tokens) const {
    std::vector<int32_t> out;
    if (add_special_tokens && add_bos_ && bos_id_ >= 0) out.push_back(bos_id_);
    size_t start = 0, i = 0;
    while (i < text.size()) {
        bool hit = false;
        for (const auto& a : added_) {
            if (!a.first.empty() && text.compare(i, a.first.size(), a.first) == 0) {
                encode_plain(text.substr(start, i - start), out);
                out.push_back(a.second);
                i += a.first.size();
                start = i;
                hit = true;
                break;
            }
        }
        if (!hit) ++i;
    }
    encode_plain(text.substr(start), out);
    return out;
}

std::string Tokenizer::id_to_bytes(int32_t id) const {
    const std::string& piece = id_to_piece(id);
    if (piece.empty()) return "";
    if (is_special(id)) return piece;
    for (const auto& a : added_)
        if (a.second == id) return piece;
    std::string o;
    if (byte_level_) {
        for (size_t i = 0; i < piece.size();) {
            const size_t s = i;
            next_cp(piece, i);
            auto it = uni_to_byte_.find(piece.substr(s, i - s));
            if (it != uni_to_byte_.end()) o += static_cast<char>(it->second);
            else o += piece.substr(s, i - s);
        }
        return o;
    }
    if (piece.size() == 6 && piece[0] == '<' && piece[1] == '0' && piece[2] == 'x' && piece[5] == '>') {
        o += static_cast<char>(std::stoi(piece.substr(3, 2), nullptr, 16));
        return o;
    }
    for (size_t i = 0; i < piece.size();) {
        if (piece.compare(i, 3, "\xE2\x96\x81") == 0) { o += ' '; i += 3; }
        else o += piece[i++];
    }
    return o;
}

std::string Tokenizer::decode(const std::vector<int32_t>& ids, bool skip_special_tokens) const {
    std::string o;
    for (int32_t id : ids) {
        if (skip_special_tokens && is_special(id)) continue;
        o += id_to_bytes(id);
    }
    if (!byte_level_ && prepend_metaspace_ && !o.empty() && o[0] == ' ') o.erase(0, 1);
    return o;
}

// ---- chat template ------------------------------------------------------------------------------
ChatTemplate ChatTemplate::from_template_text(const std::string& t, const std::string& bos) {
    ChatTemplate c;
    c.source_ = t;
    c.bos_ = bos;
    if (t.find("<|im_start|>") != std::string::npos) c.family_ = Family::kChatML;
    else if (t.find("<|start_header_id|>") != std::string::npos) c.family_ = Family::kLlama3;
    else if (t.find("[INST]") != std::string::npos) c.family_ = Family::kLlama2;
    else if (t.empty()) c.family_ = Family::kChatML;
    else c.family_ = Family::kPlain;
    if (t.find("You are a helpful assistant") != std::string::npos) c.default_system_ = "You are a helpful assistant.";
    if (t.find("You are Qwen, created by Alibaba Cloud") != std::string::npos)
        c.default_system_ = "You are Qwen, created by Alibaba Cloud. You are a helpful assistant.";
    return c;
}

ChatTemplate ChatTemplate::load(const std::string& model_dir) {
    std::string tmpl, bos;
    std::ifstream f(model_dir + "/tokenizer_config.json");
    if (f) {
        std::ostringstream ss;
        ss << f.rdbuf();
        const Json cfg = Json::parse(ss.str());
        tmpl = cfg["chat_template"].as_string();
        const Json& b = cfg["bos_token"];
        bos = b.is_string() ? b.as_string() : b["content"].as_string();
    }
    std::ifstream g(model_dir + "/chat_template.jinja");
    if (tmpl.empty() && g) {
        std::ostringstream ss;
        ss << g.rdbuf();
        tmpl = ss.str();
    }
    return from_template_text(tmpl, bos);
}

std::string ChatTemplate::apply(const std::vector<ChatMessage>& msgs, bool add_generation_prompt, bool enable_thinking) const {
    std::string o;
    switch (family_) {
        case Family::kChatML: {
            const bool has_system = !msgs.empty() && msgs[0].role == "system";
            if (!has_system && !default_system_.empty()) o += "<|im_start|>system\n" + default_system_ + "<|im_end|>\n";
            for (const auto& m : msgs) o += "<|im_start|>" + m.role + "\n" + m.content + "<|im_end|>\n";
            if (add_generation_prompt) {
                o += "<|im_start|>assistant\n";
                if (!enable_thinking && source_.find("enable_thinking") != std::string::npos) o += "<think>\n\n</think>\n\n";
            }
            break;
        }
        case Family::kLlama3: {
            o += bos_.empty() ? "<|begin_of_text|>" : bos_;
            for (const auto& m : msgs) o += "<|start_header_id|>" + m.role + "<|end_header_id|>\n\n" + m.content + "<|eot_id|>";
            if (add_generation_prompt) o += "<|start_header_id|>assistant<|end_header_id|>\n\n";
            break;
        }
        case Family::kLlama2: {
            std::string system;
            size_t i = 0;
            if (!msgs.empty() && msgs[0].role == "system") { system = msgs[0].content; i = 1; }
            bool first = true;
            for (; i < msgs.size(); ++i) {
                const auto& m = msgs[i];
                if (m.role == "user") {
                    o += (bos_.empty() ? "<s>" : bos_) + "[INST] ";
                    if (first && !system.empty()) o += "<<SYS>>\n" + system + "\n<</SYS>>\n\n";
                    o += m.content + " [/INST]";
                    first = false;
                } else {
                    o += " " + m.content + " </s>";
                }
            }
            break;
        }
        case Family::kPlain:
            for (const auto& m : msgs) o += m.role + ": " + m.content + "\n";
            if (add_generation_prompt) o += "assistant: ";
            break;
    }
    return o;
}

}  // namespace telb
