// A SentencePiece runtime of the data pipeline: reads a serialized model (the protobuf wire format is parsed here,
// no protobuf library), normalizes text with the model's precompiled character map, segments it with the unigram
// (Viterbi, n-best, lattice sampling), BPE (merge agenda, BPE-dropout), character or word algorithm, and maps ids
// back to text. Encoders produce int64 tensors directly, so a tokenizer can run as a pipeline `map` step on the
// native worker threads without the interpreter lock.
//
// Behaviour follows the published SentencePiece algorithms (cf. fairseq2n `data/text/sentencepiece/`, which wraps the
// upstream library): whitespace is escaped as U+2581, a dummy prefix is added, user-defined symbols are matched before
// normalization, runs of unknown characters merge into one unknown token (or fall back to byte pieces), control
// symbols are never produced from text and decode to nothing.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <fstream>
#include <functional>
#include <limits>
#include <queue>
#include <random>
#include <sstream>
#include <unordered_map>

#include "extras.h"

namespace fs2d {

namespace {

constexpr const char* kSpace = "\xe2\x96\x81";  // U+2581
constexpr size_t kSpaceLen = 3;
constexpr float kUnkPenalty = 10.0f;

enum PieceType { NORMAL = 1, UNKNOWN = 2, CONTROL = 3, USER_DEFINED = 4, UNUSED = 5, BYTE = 6 };
enum ModelType { UNIGRAM = 1, BPE = 2, WORD = 3, CHAR = 4 };

// ---------------------------------------------------------------------------------------------------------------
// protobuf wire format
// ---------------------------------------------------------------------------------------------------------------
struct Wire {
    const uint8_t* p;
    const uint8_t* end;

    bool done() const { return p >= end; }

    uint64_t varint() {
        uint64_t v = 0;
        for (int shift = 0; shift < 64; shift += 7) {
            if (p >= end) throw std::invalid_argument("The SentencePiece model is truncated.");
            uint8_t b = *p++;
            v |= static_cast<uint64_t>(b & 0x7f) << shift;
            if (!(b & 0x80)) return v;
        }
        throw std::invalid_argument("The SentencePiece model holds a malformed integer.");
    }

    std::string_view bytes() {
        uint64_t n = varint();
        if (n > static_cast<uint64_t>(end - p)) throw std::invalid_argument("The SentencePiece model is truncated.");
        std::string_view s(reinterpret_cast<const char*>(p), n);
        p += n;
        return s;
    }

    float f32() {
        if (end - p < 4) throw std::invalid_argument("The SentencePiece model is truncated.");
        float f;
        std::memcpy(&f, p, 4);
        p += 4;
        return f;
    }

    void skip(int wire_type) {
        switch (wire_type) {
            case 0: varint(); break;
            case 1:
                if (end - p < 8) throw std::invalid_argument("The SentencePiece model is truncated.");
                p += 8;
                break;
            case 2: bytes(); break;
            case 5:
                if (end - p < 4) throw std::invalid_argument("The SentencePiece model is truncated.");
                p += 4;
                break;
            default: throw std::invalid_argument("The SentencePiece model uses an unsupported wire type.");
        }
    }
};

Wire wire_of(std::string_view s) {
    auto* b = reinterpret_cast<const uint8_t*>(s.data());
    return Wire{b, b + s.size()};
}

inline size_t one_char_len(char c) {
    static const char len[] = "\1\1\1\1\1\1\1\1\1\1\1\1\2\2\3\4";
    return static_cast<size_t>(len[(static_cast<uint8_t>(c)) >> 4]);
}

// Length of the valid UTF-8 character at the head of `s`, or 0.
size_t valid_utf8_len(std::string_view s) {
    if (s.empty()) return 0;
    auto b = [&](size_t i) { return static_cast<uint8_t>(s[i]); };
    auto trail = [&](size_t i) { return i < s.size() && (b(i) & 0xc0) == 0x80; };
    uint8_t c = b(0);
    if (c < 0x80) return 1;
    if (c >= 0xc2 && c <= 0xdf) return trail(1) ? 2 : 0;
    if (c >= 0xe0 && c <= 0xef) {
        if (!trail(1) || !trail(2)) return 0;
        uint32_t cp = ((c & 0x0f) << 12) | ((b(1) & 0x3f) << 6) | (b(2) & 0x3f);
        if (cp < 0x800 || (cp >= 0xd800 && cp <= 0xdfff)) return 0;
        return 3;
    }
    if (c >= 0xf0 && c <= 0xf4) {
        if (!trail(1) || !trail(2) || !trail(3)) return 0;
        uint32_t cp = ((c & 0x07) << 18) | ((b(1) & 0x3f) << 12) | ((b(2) & 0x3f) << 6) | (b(3) & 0x3f);
        if (cp < 0x10000 || cp > 0x10ffff) return 0;
        return 4;
    }
    return 0;
}

// ---------------------------------------------------------------------------------------------------------------
// A byte trie over a sorted edge table: the children of a node are contiguous and ordered by label.
// ---------------------------------------------------------------------------------------------------------------
class ByteTrie {
public:
    void build(std::vector<std::pair<std::string, int>> keys) {
        std::sort(keys.begin(), keys.end());
        nodes_.clear();
        edges_.clear();
        nodes_.push_back(Node{});
        // breadth-first over key ranges so that every node's edges are contiguous
        struct Item { int node; size_t lo, hi, depth; };
        std::queue<Item> work;
        work.push(Item{0, 0, keys.size(), 0});
        while (!work.empty()) {
            Item it = work.front();
            work.pop();
            size_t lo = it.lo;
            if (lo < it.hi && keys[lo].first.size() == it.depth) {
                nodes_[it.node].value = keys[lo].second;
                ++lo;
            }
            nodes_[it.node].first_edge = static_cast<int>(edges_.size());
            std::vector<Item> children;
            size_t i = lo;
            while (i < it.hi) {
                uint8_t label = static_cast<uint8_t>(keys[i].first[it.depth]);
                size_t j = i;
                while (j < it.hi && static_cast<uint8_t>(keys[j].first[it.depth]) == label) ++j;
                int child = static_cast<int>(nodes_.size());
                nodes_.push_back(Node{});
                edges_.push_back(Edge{label, child});
                children.push_back(Item{child, i, j, it.depth + 1});
                i = j;
            }
            nodes_[it.node].num_edges = static_cast<int>(edges_.size()) - nodes_[it.node].first_edge;
            for (auto& c : children) work.push(c);
        }
    }

    bool empty() const { return nodes_.size() <= 1; }

    // -1 when there is no such child
    int step(int node, uint8_t label) const {
        const Node& n = nodes_[node];
        int lo = n.first_edge, hi = n.first_edge + n.num_edges;
        while (lo < hi) {
            int mid = (lo + hi) >> 1;
            if (edges_[mid].label < label) lo = mid + 1;
            else hi = mid;
        }
        if (lo < n.first_edge + n.num_edges && edges_[lo].label == label) return edges_[lo].child;
        return -1;
    }

    int value(int node) const { return nodes_[node].value; }

    int find(std::string_view key) const {
        int node = 0;
        for (char c : key) {
            node = step(node, static_cast<uint8_t>(c));
            if (node < 0) return -1;
        }
        return nodes_[node].value;
    }

    // Longest key that is a prefix of `s`: its length (0 if none).
    size_t longest_prefix(std::string_view s) const {
        size_t best = 0;
        int node = 0;
        for (size_t i = 0; i < s.size(); ++i) {
            node = step(node, static_cast<uint8_t>(s[i]));
            if (node < 0) break;
            if (nodes_[node].value >= 0) best = i + 1;
        }
        return best;
    }

private:
    struct Node { int value = -1; int first_edge = 0; int num_edges = 0; };
    struct Edge { uint8_t label; int child; };
    std::vector<Node> nodes_;
    std::vector<Edge> edges_;
};

// ---------------------------------------------------------------------------------------------------------------
// The precompiled character map: a double-array trie (uint32 units) followed by a pool of NUL-terminated
// replacement strings. Unit layout: bit 8 = "has leaf", bit 9 = offset scale, bits 10.. = offset, low byte +
// bit 31 = label; a leaf unit's low 31 bits are the value (an offset into the pool).
// ---------------------------------------------------------------------------------------------------------------
class CharsMap {
public:
    void load(std::string_view blob) {
        units_.clear();
        pool_.clear();
        if (blob.empty()) return;
        if (blob.size() < 4) throw std::invalid_argument("The character map of the SentencePiece model is truncated.");
        uint32_t trie_bytes;
        std::memcpy(&trie_bytes, blob.data(), 4);
        if (trie_bytes > blob.size() - 4 || trie_bytes % 4 != 0 || trie_bytes < 1024)
            throw std::invalid_argument("The character map of the SentencePiece model is malformed.");
        units_.resize(trie_bytes / 4);
        std::memcpy(units_.data(), blob.data() + 4, trie_bytes);
        pool_.assign(blob.data() + 4 + trie_bytes, blob.size() - 4 - trie_bytes);
        pool_.push_back('\0');
    }

    bool empty() const { return units_.empty(); }

    // Longest rule that matches a prefix of `s`: (replacement, matched bytes); matched == 0 when none applies.
    std::pair<std::string_view, size_t> longest(std::string_view s) const {
        size_t best_len = 0;
        uint32_t best_val = 0;
        size_t pos = 0;
        uint32_t unit = units_[0];
        pos ^= offset(unit);
        for (size_t i = 0; i < s.size(); ++i) {
            uint8_t c = static_cast<uint8_t>(s[i]);
            pos ^= c;
            if (pos >= units_.size()) break;
            unit = units_[pos];
            if ((unit & ((1u << 31) | 0xffu)) != c) break;
            pos ^= offset(unit);
            if ((unit >> 8) & 1u) {
                if (pos >= units_.size()) break;
                best_len = i + 1;
                best_val = units_[pos] & ((1u << 31) - 1);
            }
        }
        if (best_len == 0 || best_val >= pool_.size()) return {std::string_view(), 0};
        return {std::string_view(pool_.c_str() + best_val), best_len};
    }

private:
    static size_t offset(uint32_t unit) { return static_cast<size_t>((unit >> 10) << ((unit & (1u << 9)) >> 6)); }
    std::vector<uint32_t> units_;
    std::string pool_;
};

struct Piece {
    std::string text;
    float score = 0.f;
    int type = NORMAL;
};

}  // namespace

// ---------------------------------------------------------------------------------------------------------------
// the model
// ---------------------------------------------------------------------------------------------------------------
struct SentencePieceModel::Impl {
    std::vector<Piece> pieces;
    int model_type = UNIGRAM;
    bool byte_fallback = false;
    bool treat_ws_as_suffix = false;
    std::string unk_piece = "<unk>", bos_piece = "<s>", eos_piece = "</s>", pad_piece = "<pad>";
    std::string unk_surface = " \xe2\x81\x87 ";
    bool add_dummy_prefix = true, remove_extra_ws = true, escape_ws = true;
    CharsMap charsmap;

    ByteTrie trie;          // NORMAL, USER_DEFINED and UNUSED pieces
    ByteTrie user_trie;     // USER_DEFINED pieces (matched before normalization and never split)
    std::unordered_map<std::string, int> reserved;  // CONTROL, UNKNOWN and BYTE pieces
    int unk_id = -1;
    float min_score = 0.f, max_score = 0.f;
    int byte_ids[256];

    void parse(std::string_view proto);
    void index();

    int piece_to_id(std::string_view piece) const {
        auto it = reserved.find(std::string(piece));
        if (it != reserved.end()) return it->second;
        int id = trie.find(piece);
        return id >= 0 ? id : unk_id;
    }

    int control_id(const std::string& piece) const {
        int id = piece_to_id(piece);
        return (id >= 0 && pieces[id].type == CONTROL) ? id : -1;
    }

    // -- normalization --------------------------------------------------------------------------------------
    std::pair<std::string_view, size_t> normalize_prefix(std::string_view in) const {
        static const char kReplacement[] = "\xef\xbf\xbd";
        if (!user_trie.empty()) {
            size_t n = user_trie.longest_prefix(in);
            if (n > 0) return {in.substr(0, n), n};
        }
        if (!charsmap.empty()) {
            auto r = charsmap.longest(in);
            if (r.second > 0) return r;
        }
        size_t n = valid_utf8_len(in);
        if (n == 0) return {std::string_view(kReplacement, 3), 1};
        return {in.substr(0, n), n};
    }

    std::string normalize(std::string_view in) const {
        std::string out;
        if (remove_extra_ws) {
            while (!in.empty()) {
                auto p = normalize_prefix(in);
                if (p.first != " ") break;
                in.remove_prefix(p.second);
            }
        }
        if (in.empty()) return out;
        out.reserve(in.size() * 3 / 2 + 8);
        auto add_ws = [&] {
            if (escape_ws) out.append(kSpace, kSpaceLen);
            else out.push_back(' ');
        };
        if (!treat_ws_as_suffix && add_dummy_prefix) add_ws();
        bool prev_space = remove_extra_ws;
        while (!in.empty()) {
            auto p = normalize_prefix(in);
            std::string_view sp = p.first;
            while (prev_space && !sp.empty() && sp.front() == ' ') sp.remove_prefix(1);
            if (!sp.empty()) {
                for (char c : sp) {
                    if (escape_ws && c == ' ') out.append(kSpace, kSpaceLen);
                    else out.push_back(c);
                }
                prev_space = sp.back() == ' ';
            }
            in.remove_prefix(p.second);
            if (!remove_extra_ws) prev_space = false;
        }
        if (remove_extra_ws) {
            std::string_view space = escape_ws ? std::string_view(kSpace, kSpaceLen) : std::string_view(" ", 1);
            while (out.size() >= space.size() && std::string_view(out).substr(out.size() - space.size()) == space)
                out.resize(out.size() - space.size());
        }
        if (treat_ws_as_suffix && add_dummy_prefix) add_ws();
        return out;
    }

    // user-defined symbol or one character
    size_t symbol_len(std::string_view s, bool* is_user = nullptr) const {
        if (!user_trie.empty()) {
            size_t n = user_trie.longest_prefix(s);
            if (n > 0) {
                if (is_user) *is_user = true;
                return n;
            }
        }
        if (is_user) *is_user = false;
        return std::min(one_char_len(s[0]), s.size());
    }

    using Seg = std::pair<std::string_view, int>;

    // -- unigram --------------------------------------------------------------------------------------------
    std::vector<Seg> unigram_viterbi(std::string_view norm) const {
        struct Best { int id = -1; float score = 0.f; int start = -1; };
        const size_t n = norm.size();
        std::vector<Best> best(n + 1);
        const float unk_score = min_score - kUnkPenalty;
        size_t start = 0;
        while (start < n) {
            const float here = best[start].score;
            bool has_single = false;
            const size_t mblen = std::min(one_char_len(norm[start]), n - start);
            int node = 0;
            for (size_t pos = start; pos < n;) {
                node = trie.step(node, static_cast<uint8_t>(norm[pos]));
                if (node < 0) break;
                ++pos;
                int id = trie.value(node);
                if (id < 0) continue;
                const Piece& pc = pieces[id];
                if (pc.type == UNUSED) continue;
                const size_t length = pos - start;
                const float score = pc.type == USER_DEFINED ? length * max_score - 0.1f : pc.score;
                const float cand = score + here;
                Best& t = best[pos];
                if (t.start == -1 || cand > t.score) {
                    t.score = cand;
                    t.start = static_cast<int>(start);
                    t.id = id;
                }
                if (!has_single && length == mblen) has_single = true;
            }
            if (!has_single) {
                Best& t = best[start + mblen];
                const float cand = unk_score + here;
                if (t.start == -1 || cand > t.score) {
                    t.score = cand;
                    t.start = static_cast<int>(start);
                    t.id = unk_id;
                }
            }
            start += mblen;
        }
        std::vector<Seg> out;
        size_t end = n;
        while (end > 0) {
            const Best& b = best[end];
            out.emplace_back(norm.substr(b.start, end - b.start), b.id);
            end = static_cast<size_t>(b.start);
        }
        std::reverse(out.begin(), out.end());
        return out;
    }

    struct LatNode { int pos; int len; int id; float score; };

    // All segmentation candidates: nodes grouped by their end position.
    void lattice(std::string_view norm, std::vector<LatNode>& nodes, std::vector<std::vector<int>>& ends_at,
                 std::vector<std::vector<int>>& begins_at) const {
        const size_t n = norm.size();
        ends_at.assign(n + 1, {});
        begins_at.assign(n + 1, {});
        const float unk_score = min_score - kUnkPenalty;
        size_t start = 0;
        while (start < n) {
            const size_t mblen = std::min(one_char_len(norm[start]), n - start);
            bool has_single = false;
            int node = 0;
            for (size_t pos = start; pos < n;) {
                node = trie.step(node, static_cast<uint8_t>(norm[pos]));
                if (node < 0) break;
                ++pos;
                int id = trie.value(node);
                if (id < 0 || pieces[id].type == UNUSED) continue;
                const int length = static_cast<int>(pos - start);
                const float score = pieces[id].type == USER_DEFINED ? length * max_score - 0.1f : pieces[id].score;
                nodes.push_back(LatNode{static_cast<int>(start), length, id, score});
                if (static_cast<size_t>(length) == mblen) has_single = true;
            }
            if (!has_single) nodes.push_back(LatNode{static_cast<int>(start), static_cast<int>(mblen), unk_id, unk_score});
            start += mblen;
        }
        for (size_t i = 0; i < nodes.size(); ++i) {
            ends_at[nodes[i].pos + nodes[i].len].push_back(static_cast<int>(i));
            begins_at[nodes[i].pos].push_back(static_cast<int>(i));
        }
    }

    static float log_sum_exp(float a, float b, bool init) {
        if (init) return b;
        const float hi = std::max(a, b), lo = std::min(a, b);
        if (hi > lo + 50.f) return hi;
        return hi + std::log1p(std::exp(lo - hi));
    }

    // Forward filtering, backward sampling over the lattice with inverse temperature `theta`.
    std::vector<Seg> unigram_sample(std::string_view norm, float theta, std::mt19937_64& rng) const {
        std::vector<LatNode> nodes;
        std::vector<std::vector<int>> ends_at, begins_at;
        lattice(norm, nodes, ends_at, begins_at);
        const size_t n = norm.size();
        // alpha[pos]: log of the total weight of all paths that cover [0, pos)
        std::vector<float> alpha(n + 1, 0.f);
        std::vector<char> reach(n + 1, 0);
        reach[0] = 1;
        for (size_t pos = 1; pos <= n; ++pos) {
            bool init = true;
            for (int k : ends_at[pos]) {
                const LatNode& nd = nodes[k];
                if (!reach[nd.pos]) continue;
                alpha[pos] = log_sum_exp(alpha[pos], alpha[nd.pos] + theta * nd.score, init);
                init = false;
            }
            reach[pos] = !init;
        }
        std::vector<Seg> out;
        std::uniform_real_distribution<double> uni(0.0, 1.0);
        size_t end = n;
        while (end > 0) {
            std::vector<double> w;
            std::vector<int> cand;
            double total = 0.0;
            for (int k : ends_at[end]) {
                const LatNode& nd = nodes[k];
                if (!reach[nd.pos]) continue;
                double p = std::exp(static_cast<double>(alpha[nd.pos] + theta * nd.score - alpha[end]));
                w.push_back(p);
                cand.push_back(k);
                total += p;
            }
            double r = uni(rng) * total;
            size_t pick = 0;
            for (; pick + 1 < w.size(); ++pick) {
                r -= w[pick];
                if (r <= 0.0) break;
            }
            const LatNode& nd = nodes[cand[pick]];
            out.emplace_back(norm.substr(nd.pos, nd.len), nd.id);
            end = static_cast<size_t>(nd.pos);
        }
        std::reverse(out.begin(), out.end());
        return out;
    }

    // The `nbest` highest-scoring segmentations (backward A* with the exact forward Viterbi score as heuristic).
    std::vector<std::pair<std::vector<Seg>, float>> unigram_nbest(std::string_view norm, size_t nbest) const {
        std::vector<LatNode> nodes;
        std::vector<std::vector<int>> ends_at, begins_at;
        lattice(norm, nodes, ends_at, begins_at);
        const size_t n = norm.size();
        const float ninf = -std::numeric_limits<float>::infinity();
        std::vector<float> fwd(n + 1, ninf);   // best score of a path covering [0, pos)
        fwd[0] = 0.f;
        for (size_t pos = 1; pos <= n; ++pos)
            for (int k : ends_at[pos])
                if (fwd[nodes[k].pos] != ninf) fwd[pos] = std::max(fwd[pos], fwd[nodes[k].pos] + nodes[k].score);
        struct Hyp { int node; int next; float gx; float fx; };   // `next`: index of the hypothesis to the right
        std::vector<Hyp> hyps;
        auto cmp = [&](int a, int b) { return hyps[a].fx < hyps[b].fx; };
        std::priority_queue<int, std::vector<int>, decltype(cmp)> agenda(cmp);
        std::vector<std::pair<std::vector<Seg>, float>> results;
        for (int k : ends_at[n]) {
            if (fwd[nodes[k].pos] == ninf) continue;
            hyps.push_back(Hyp{k, -1, nodes[k].score, nodes[k].score + fwd[nodes[k].pos]});
            agenda.push(static_cast<int>(hyps.size()) - 1);
        }
        constexpr size_t kMaxAgenda = 100000;
        while (!agenda.empty() && results.size() < nbest && hyps.size() < kMaxAgenda) {
            int h = agenda.top();
            agenda.pop();
            const LatNode& nd = nodes[hyps[h].node];
            if (nd.pos == 0) {
                std::vector<Seg> segs;
                for (int c = h; c != -1; c = hyps[c].next) {
                    const LatNode& x = nodes[hyps[c].node];
                    segs.emplace_back(norm.substr(x.pos, x.len), x.id);
                }
                results.emplace_back(std::move(segs), hyps[h].gx);
                continue;
            }
            for (int k : ends_at[nd.pos]) {
                if (fwd[nodes[k].pos] == ninf) continue;
                float gx = hyps[h].gx + nodes[k].score;
                hyps.push_back(Hyp{k, h, gx, gx + fwd[nodes[k].pos]});
                agenda.push(static_cast<int>(hyps.size()) - 1);
            }
        }
        return results;
    }

    // -- BPE ------------------------------------------------------------------------------------------------
    std::vector<Seg> bpe(std::string_view norm, float dropout, std::mt19937_64* rng) const {
        struct Symbol { int prev, next; bool freeze; std::string_view piece; };
        struct Pair { int left, right; float score; size_t size; };
        auto worse = [](const Pair& a, const Pair& b) {
            return a.score < b.score || (a.score == b.score && a.left > b.left);
        };
        std::priority_queue<Pair, std::vector<Pair>, decltype(worse)> agenda(worse);
        std::vector<Symbol> symbols;
        std::unordered_map<std::string_view, std::pair<std::string_view, std::string_view>> rev_merge;

        std::string_view rest = norm;
        int index = 0;
        while (!rest.empty()) {
            Symbol s;
            size_t n = symbol_len(rest, &s.freeze);
            s.piece = rest.substr(0, n);
            s.prev = index == 0 ? -1 : index - 1;
            rest.remove_prefix(n);
            s.next = rest.empty() ? -1 : index + 1;
            ++index;
            symbols.push_back(s);
        }
        std::vector<Seg> out;
        if (symbols.empty()) return out;

        auto maybe_add = [&](int left, int right) {
            if (left == -1 || right == -1 || symbols[left].freeze || symbols[right].freeze) return;
            std::string_view piece(symbols[left].piece.data(), symbols[left].piece.size() + symbols[right].piece.size());
            int id = trie.find(piece);
            if (id < 0) return;
            agenda.push(Pair{left, right, pieces[id].score, piece.size()});
            if (pieces[id].type == UNUSED) rev_merge[piece] = {symbols[left].piece, symbols[right].piece};
        };
        for (size_t i = 1; i < symbols.size(); ++i) maybe_add(static_cast<int>(i) - 1, static_cast<int>(i));

        std::uniform_real_distribution<double> uni(0.0, 1.0);
        while (!agenda.empty()) {
            Pair top = agenda.top();
            agenda.pop();
            Symbol& l = symbols[top.left];
            Symbol& r = symbols[top.right];
            if (l.piece.empty() || r.piece.empty() || l.piece.size() + r.piece.size() != top.size) continue;
            if (dropout > 0.f && rng != nullptr && uni(*rng) < dropout) continue;
            l.piece = std::string_view(l.piece.data(), l.piece.size() + r.piece.size());
            l.next = r.next;
            if (r.next >= 0) symbols[r.next].prev = top.left;
            r.piece = std::string_view();
            maybe_add(l.prev, top.left);
            maybe_add(top.left, l.next);
        }

        std::function<void(std::string_view)> resegment = [&](std::string_view w) {
            int id = piece_to_id(w);
            if (id < 0 || pieces[id].type != UNUSED) {
                out.emplace_back(w, id);
                return;
            }
            auto it = rev_merge.find(w);
            if (it == rev_merge.end()) {
                out.emplace_back(w, id);
                return;
            }
            resegment(it->second.first);
            resegment(it->second.second);
        };
        for (int i = 0; i != -1; i = symbols[i].next) resegment(symbols[i].piece);
        return out;
    }

    // -- character and word models --------------------------------------------------------------------------
    std::vector<Seg> chars(std::string_view norm) const {
        std::vector<Seg> out;
        while (!norm.empty()) {
            size_t n = symbol_len(norm);
            out.emplace_back(norm.substr(0, n), piece_to_id(norm.substr(0, n)));
            norm.remove_prefix(n);
        }
        return out;
    }

    std::vector<Seg> words(std::string_view norm) const {
        // a word starts at every whitespace symbol (or ends with it when whitespace is a suffix)
        std::vector<Seg> out;
        std::vector<size_t> cuts{0};
        std::string_view sp(kSpace, kSpaceLen);
        for (size_t i = 0; i < norm.size();) {
            size_t n = std::min(one_char_len(norm[i]), norm.size() - i);
            bool is_space = norm.substr(i, n) == sp;
            if (is_space && !treat_ws_as_suffix && i != 0) cuts.push_back(i);
            if (is_space && treat_ws_as_suffix && i + n < norm.size()) cuts.push_back(i + n);
            i += n;
        }
        cuts.push_back(norm.size());
        for (size_t k = 0; k + 1 < cuts.size(); ++k) {
            std::string_view w = norm.substr(cuts[k], cuts[k + 1] - cuts[k]);
            if (!w.empty()) out.emplace_back(w, piece_to_id(w));
        }
        return out;
    }

    // -- shared post-processing -----------------------------------------------------------------------------
    std::vector<std::pair<std::string, int>> finish(const std::vector<Seg>& segs) const {
        std::vector<std::pair<std::string, int>> out;
        out.reserve(segs.size());
        bool prev_unk = false;
        for (const Seg& s : segs) {
            if (s.first.empty()) throw std::runtime_error("The SentencePiece segmentation produced an empty piece.");
            const bool is_unk = s.second == unk_id;
            if (is_unk && byte_fallback) {
                for (char c : s.first) {
                    uint8_t b = static_cast<uint8_t>(c);
                    out.emplace_back(pieces[byte_ids[b]].text, byte_ids[b]);
                }
            } else if (is_unk && prev_unk) {
                out.back().first.append(s.first);
            } else {
                out.emplace_back(std::string(s.first), s.second);
            }
            prev_unk = is_unk;
        }
        return out;
    }

    std::vector<Seg> segment(std::string_view norm, const SamplingOptions* sampling, std::mt19937_64* rng,
                             std::vector<std::pair<std::vector<Seg>, float>>* scratch) const {
        if (norm.empty()) return {};
        switch (model_type) {
            case UNIGRAM:
                if (sampling != nullptr && rng != nullptr) {
                    if (sampling->nbest_size < 0) return unigram_sample(norm, sampling->alpha, *rng);
                    if (sampling->nbest_size > 1) {
                        *scratch = unigram_nbest(norm, static_cast<size_t>(sampling->nbest_size));
                        if (scratch->empty()) return unigram_viterbi(norm);
                        std::vector<double> w;
                        for (auto& r : *scratch) w.push_back(std::exp(static_cast<double>(sampling->alpha * (r.second - (*scratch)[0].second))));
                        std::discrete_distribution<size_t> pick(w.begin(), w.end());
                        return (*scratch)[pick(*rng)].first;
                    }
                }
                return unigram_viterbi(norm);
            case BPE:
                return bpe(norm, sampling != nullptr ? sampling->alpha : 0.f, sampling != nullptr ? rng : nullptr);
            case CHAR: return chars(norm);
            case WORD: return words(norm);
            default: throw std::runtime_error("The SentencePiece model has an unknown model type.");
        }
    }
};

void SentencePieceModel::Impl::parse(std::string_view proto) {
    Wire w = wire_of(proto);
    while (!w.done()) {
        uint64_t key = w.varint();
        int field = static_cast<int>(key >> 3), wt = static_cast<int>(key & 7);
        if (field == 1 && wt == 2) {
            Wire pw = wire_of(w.bytes());
            Piece pc;
            while (!pw.done()) {
                uint64_t k = pw.varint();
                int f = static_cast<int>(k >> 3), t = static_cast<int>(k & 7);
                if (f == 1 && t == 2) pc.text = std::string(pw.bytes());
                else if (f == 2 && t == 5) pc.score = pw.f32();
                else if (f == 3 && t == 0) pc.type = static_cast<int>(pw.varint());
                else pw.skip(t);
            }
            pieces.push_back(std::move(pc));
        } else if (field == 2 && wt == 2) {
            Wire tw = wire_of(w.bytes());
            while (!tw.done()) {
                uint64_t k = tw.varint();
                int f = static_cast<int>(k >> 3), t = static_cast<int>(k & 7);
                if (f == 3 && t == 0) model_type = static_cast<int>(tw.varint());
                else if (f == 24 && t == 0) treat_ws_as_suffix = tw.varint() != 0;
                else if (f == 35 && t == 0) byte_fallback = tw.varint() != 0;
                else if (f == 44 && t == 2) unk_surface = std::string(tw.bytes());
                else if (f == 45 && t == 2) unk_piece = std::string(tw.bytes());
                else if (f == 46 && t == 2) bos_piece = std::string(tw.bytes());
                else if (f == 47 && t == 2) eos_piece = std::string(tw.bytes());
                else if (f == 48 && t == 2) pad_piece = std::string(tw.bytes());
                else tw.skip(t);
            }
        } else if (field == 3 && wt == 2) {
            Wire nw = wire_of(w.bytes());
            while (!nw.done()) {
                uint64_t k = nw.varint();
                int f = static_cast<int>(k >> 3), t = static_cast<int>(k & 7);
                if (f == 2 && t == 2) charsmap.load(nw.bytes());
                else if (f == 3 && t == 0) add_dummy_prefix = nw.varint() != 0;
                else if (f == 4 && t == 0) remove_extra_ws = nw.varint() != 0;
                else if (f == 5 && t == 0) escape_ws = nw.varint() != 0;
                else nw.skip(t);
            }
        } else {
            w.skip(wt);
        }
    }
    if (pieces.empty()) throw std::invalid_argument("The SentencePiece model holds no pieces.");
}

void SentencePieceModel::Impl::index() {
    std::vector<std::pair<std::string, int>> normal, user;
    reserved.clear();
    unk_id = -1;
    std::fill(std::begin(byte_ids), std::end(byte_ids), -1);
    min_score = std::numeric_limits<float>::max();
    max_score = std::numeric_limits<float>::lowest();
    for (size_t i = 0; i < pieces.size(); ++i) {
        const Piece& pc = pieces[i];
        if (pc.text.empty()) throw std::invalid_argument("The SentencePiece model holds an empty piece.");
        const int id = static_cast<int>(i);
        const bool in_trie = pc.type == NORMAL || pc.type == USER_DEFINED || pc.type == UNUSED;
        if (in_trie) normal.emplace_back(pc.text, id);
        else if (!reserved.emplace(pc.text, id).second)
            throw std::invalid_argument("The SentencePiece model defines the piece '" + pc.text + "' twice.");
        if (pc.type == USER_DEFINED) user.emplace_back(pc.text, id);
        if (pc.type == UNKNOWN) {
            if (unk_id >= 0) throw std::invalid_argument("The SentencePiece model defines the unknown piece twice.");
            unk_id = id;
        }
        if (pc.type == NORMAL) {
            min_score = std::min(min_score, pc.score);
            max_score = std::max(max_score, pc.score);
        }
        if (pc.type == BYTE) {
            unsigned v = 0;
            if (pc.text.size() == 6 && std::sscanf(pc.text.c_str(), "<0x%02X>", &v) == 1) byte_ids[v & 0xff] = id;
        }
    }
    if (unk_id < 0) throw std::invalid_argument("The SentencePiece model defines no unknown piece.");
    if (min_score > max_score) min_score = max_score = 0.f;
    {
        auto sorted = normal;
        std::sort(sorted.begin(), sorted.end());
        for (size_t i = 1; i < sorted.size(); ++i)
            if (sorted[i].first == sorted[i - 1].first)
                throw std::invalid_argument("The SentencePiece model defines the piece '" + sorted[i].first + "' twice.");
    }
    trie.build(std::move(normal));
    user_trie.build(std::move(user));
    if (byte_fallback)
        for (int b = 0; b < 256; ++b)
            if (byte_ids[b] < 0)
                throw std::invalid_argument("The SentencePiece model enables byte fallback, but lacks a byte piece.");
}

SentencePieceModel::SentencePieceModel(std::string_view serialized, const std::vector<std::string>& control_symbols)
    : impl_(std::make_shared<Impl>()) {
    impl_->parse(serialized);
    // Extra control symbols: "<sym>@0" is inserted at index 0 (every piece moves up by one), any other symbol that
    // the model does not hold is appended.
    for (const std::string& raw : control_symbols) {
        if (raw.empty()) continue;
        bool front = raw.size() > 2 && raw.compare(raw.size() - 2, 2, "@0") == 0;
        std::string sym = front ? raw.substr(0, raw.size() - 2) : raw;
        bool known = false;
        for (const Piece& pc : impl_->pieces)
            if (pc.text == sym) {
                known = true;
                break;
            }
        if (known) continue;
        Piece pc;
        pc.text = sym;
        pc.type = CONTROL;
        if (front) {
            impl_->pieces.insert(impl_->pieces.begin(), std::move(pc));
            impl_->pad_piece = sym;
        } else {
            impl_->pieces.push_back(std::move(pc));
        }
    }
    impl_->index();
}

SentencePieceModel SentencePieceModel::from_file(const std::string& path,
                                                 const std::vector<std::string>& control_symbols) {
    std::ifstream fp(path, std::ios::binary);
    if (!fp) throw std::runtime_error("The SentencePiece model '" + path + "' cannot be opened: No such file or directory.");
    std::stringstream ss;
    ss << fp.rdbuf();
    std::string blob = ss.str();
    return SentencePieceModel(blob, control_symbols);
}

size_t SentencePieceModel::size() const { return impl_->pieces.size(); }
int SentencePieceModel::unk_id() const { return impl_->unk_id; }
int SentencePieceModel::bos_id() const { return impl_->control_id(impl_->bos_piece); }
int SentencePieceModel::eos_id() const { return impl_->control_id(impl_->eos_piece); }
int SentencePieceModel::pad_id() const { return impl_->control_id(impl_->pad_piece); }
int SentencePieceModel::piece_to_id(std::string_view piece) const { return impl_->piece_to_id(piece); }

const std::string& SentencePieceModel::id_to_piece(int id) const {
    if (id < 0 || static_cast<size_t>(id) >= impl_->pieces.size())
        throw std::invalid_argument("`idx` must be less than vocabulary size (" + std::to_string(impl_->pieces.size()) +
                                    "), but is " + std::to_string(id) + " instead.");
    return impl_->pieces[id].text;
}

bool SentencePieceModel::is_control(int id) const {
    return id >= 0 && static_cast<size_t>(id) < impl_->pieces.size() && impl_->pieces[id].type == CONTROL;
}

std::string SentencePieceModel::normalize(std::string_view text) const { return impl_->normalize(text); }

std::vector<std::pair<std::string, int>> SentencePieceModel::encode_as_pieces(std::string_view text,
                                                                              const SamplingOptions* sampling,
                                                                              std::mt19937_64* rng) const {
    std::string norm = impl_->normalize(text);
    std::vector<std::pair<std::vector<Impl::Seg>, float>> scratch;
    return impl_->finish(impl_->segment(norm, sampling, rng, &scratch));
}

std::vector<int64_t> SentencePieceModel::encode(std::string_view text, const SamplingOptions* sampling,
                                                std::mt19937_64* rng) const {
    auto pieces = encode_as_pieces(text, sampling, rng);
    std::vector<int64_t> ids;
    ids.reserve(pieces.size());
    for (auto& p : pieces) ids.push_back(p.second);
    return ids;
}

std::vector<std::pair<std::vector<std::pair<std::string, int>>, float>> SentencePieceModel::nbest_encode(
    std::string_view text, size_t nbest) const {
    if (impl_->model_type != UNIGRAM) throw std::invalid_argument("N-best segmentation needs a unigram model.");
    std::string norm = impl_->normalize(text);
    std::vector<std::pair<std::vector<std::pair<std::string, int>>, float>> out;
    if (norm.empty()) return out;
    for (auto& r : impl_->unigram_nbest(norm, nbest)) out.emplace_back(impl_->finish(r.first), r.second);
    return out;
}

std::string SentencePieceModel::decode_pieces(const std::vector<std::pair<std::string, int>>& pieces) const {
    const Impl& m = *impl_;
    std::string text;
    std::string bytes;
    const std::string_view sp(kSpace, kSpaceLen);
    auto flush_bytes = [&] {
        std::string_view rest(bytes);
        while (!rest.empty()) {
            size_t n = valid_utf8_len(rest);
            if (n == 0) {
                text.append("\xef\xbf\xbd");
                rest.remove_prefix(1);
            } else {
                text.append(rest.substr(0, n));
                rest.remove_prefix(n);
            }
        }
        bytes.clear();
    };
    bool at_start = true;   // no text has been produced yet: leading whitespace symbols are dropped
    for (auto& [piece, id] : pieces) {
        const int type = (id >= 0 && static_cast<size_t>(id) < m.pieces.size()) ? m.pieces[id].type : NORMAL;
        if (type == BYTE) {
            unsigned v = 0;
            if (std::sscanf(piece.c_str(), "<0x%02X>", &v) == 1) bytes.push_back(static_cast<char>(v));
            continue;
        }
        if (!bytes.empty()) {
            flush_bytes();
            at_start = false;
        }
        if (type == CONTROL) continue;
        if (type == UNKNOWN) {
            text.append(piece == m.pieces[id].text ? m.unk_surface : piece);
            at_start = false;
            continue;
        }
        std::string_view w(piece);
        if (at_start && !m.treat_ws_as_suffix && (m.add_dummy_prefix || m.remove_extra_ws)) {
            if (w.substr(0, sp.size()) == sp) {
                w.remove_prefix(sp.size());
                if (!m.remove_extra_ws) at_start = false;   // only the dummy prefix goes
            }
            if (m.remove_extra_ws)
                while (w.substr(0, sp.size()) == sp) w.remove_prefix(sp.size());
        }
        if (!w.empty()) at_start = false;
        while (!w.empty()) {
            if (w.substr(0, sp.size()) == sp) {
                text.push_back(' ');
                w.remove_prefix(sp.size());
            } else {
                text.push_back(w.front());
                w.remove_prefix(1);
            }
        }
    }
    if (!bytes.empty()) flush_bytes();
    return text;
}

std::string SentencePieceModel::decode(const std::vector<int64_t>& ids) const {
    std::vector<std::pair<std::string, int>> pieces;
    pieces.reserve(ids.size());
    for (int64_t id : ids) {
        if (id < 0 || static_cast<size_t>(id) >= impl_->pieces.size())
            throw std::out_of_range("The index " + std::to_string(id) + " is outside the SentencePiece vocabulary.");
        pieces.emplace_back(impl_->pieces[id].text, static_cast<int>(id));
    }
    return decode_pieces(pieces);
}

std::string SentencePieceModel::decode_tokens(const std::vector<std::string>& tokens) const {
    std::vector<std::pair<std::string, int>> pieces;
    pieces.reserve(tokens.size());
    for (const std::string& t : tokens) pieces.emplace_back(t, impl_->piece_to_id(t));
    return decode_pieces(pieces);
}

// ---------------------------------------------------------------------------------------------------------------
// pipeline steps
// ---------------------------------------------------------------------------------------------------------------
SentencePieceEncoder::SentencePieceEncoder(SentencePieceModel model, std::vector<std::string> prefix_tokens,
                                           std::vector<std::string> suffix_tokens, bool reverse, bool enable_sampling,
                                           int nbest_size, float alpha, std::optional<at::Device> device,
                                           bool pin_memory, uint64_t seed)
    : model_(std::move(model)), reverse_(reverse), sampling_(enable_sampling), device_(device), pin_(pin_memory),
      rng_(std::make_shared<std::pair<std::mutex, std::mt19937_64>>()) {
    options_.nbest_size = nbest_size;
    options_.alpha = alpha;
    rng_->second.seed(seed);
    auto resolve = [&](const std::vector<std::string>& tokens, std::vector<int64_t>& out) {
        for (const std::string& t : tokens) {
            int id = model_.piece_to_id(t);
            if (id == model_.unk_id() && t != model_.id_to_piece(id))
                throw std::invalid_argument("The token '" + t + "' is not in the SentencePiece vocabulary.");
            out.push_back(id);
        }
    };
    resolve(prefix_tokens, prefix_);
    resolve(suffix_tokens, suffix_);
}

at::Tensor SentencePieceEncoder::encode(std::string_view text) const {
    std::vector<int64_t> ids;
    if (sampling_) {
        // one generator per encoder; worker threads draw a private stream from it so that sampling needs no lock
        std::mt19937_64 local;
        {
            std::lock_guard<std::mutex> g(rng_->first);
            local.seed(rng_->second());
        }
        ids = model_.encode(text, &options_, &local);
    } else {
        ids = model_.encode(text);
    }
    const int64_t n = static_cast<int64_t>(prefix_.size() + ids.size() + suffix_.size());
    at::Tensor t = at::empty({n}, at::TensorOptions().dtype(at::kLong).pinned_memory(pin_ && device_.has_value() && device_->is_cuda()));
    int64_t* p = t.data_ptr<int64_t>();
    int64_t* q = std::copy(prefix_.begin(), prefix_.end(), p);
    q = std::copy(ids.begin(), ids.end(), q);
    std::copy(suffix_.begin(), suffix_.end(), q);
    if (reverse_) std::reverse(p, p + n);            // the whole sequence, prefix and suffix tokens included
    if (device_.has_value() && !device_->is_cpu()) t = t.to(*device_, /*non_blocking=*/pin_);
    return t;
}

std::vector<std::string> SentencePieceEncoder::encode_as_tokens(std::string_view text) const {
    std::vector<std::string> out;
    auto pieces = model_.encode_as_pieces(text);
    for (const int64_t id : prefix_) out.push_back(model_.id_to_piece(static_cast<int>(id)));
    for (auto& p : pieces) out.push_back(std::move(p.first));
    for (const int64_t id : suffix_) out.push_back(model_.id_to_piece(static_cast<int>(id)));
    if (reverse_) std::reverse(out.begin(), out.end());
    return out;
}

Data SentencePieceEncoder::operator()(Data&& d) const {
    if (!d.is_string()) throw std::invalid_argument("The input of a SentencePiece encoder must be a string.");
    return Data(encode(d.as_string()));
}

std::string SentencePieceDecoder::decode(const at::Tensor& indices) const {
    if (indices.dim() != 1)
        throw std::invalid_argument("The input tensor must be one dimensional, but has " + std::to_string(indices.dim()) +
                                    " dimension(s) instead.");
    if (indices.scalar_type() != at::kShort && indices.scalar_type() != at::kInt && indices.scalar_type() != at::kLong)
        throw std::invalid_argument("`sp_decoder` supports only `torch.int16`, `torch.int32`, and `torch.int64` data types.");
    at::Tensor t = indices.to(at::kCPU, at::kLong).contiguous();
    const int64_t* p = t.data_ptr<int64_t>();
    std::vector<int64_t> ids(p, p + t.numel());
    if (reverse_) std::reverse(ids.begin(), ids.end());
    return model_.decode(ids);
}

Data SentencePieceDecoder::operator()(Data&& d) const {
    if (!d.is_tensor()) throw std::invalid_argument("The input of a SentencePiece decoder must be a tensor.");
    return Data(decode(d.as_tensor()));
}

}  // namespace fs2d
