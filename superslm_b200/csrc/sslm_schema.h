// Decode schemas (the SCM1 section): per schema a DFA over token ids, with one vocab-bit mask
// page per state (the tokens allowed next), sorted (token, next state) transition rows, and the
// accepting states. Restates SchemaMasksTable (include/superslm/schema_masks.h:150-384): the
// same structural checks in the same order, so an artifact the reference refuses is refused
// here, and the same Transition lookup. Host side only; the mask pages are uploaded by the
// engine and applied inside the vocab-head kernels.
#pragma once
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

namespace sslm {

constexpr uint32_t kDfaWalkUnused = 0xFFFFFFFFu;   // "no schema bound" in sequence state and save blobs

struct SchemaEntry {
	std::string name;
	uint64_t name_hash = 0;        // FNV-1a 64 of the name: what a save blob records
	uint32_t states = 0, accepting = 0, transitions = 0;
	uint64_t pages_off = 0, offsets_off = 0, accepting_off = 0, transitions_off = 0;   // into SchemaTable::bytes
	size_t device_page0 = 0;       // index of this schema's first mask page in the device array
};

class SchemaTable {
public:
	std::vector<uint8_t> bytes;    // the section, owned
	std::vector<SchemaEntry> entries;
	uint32_t vocab = 0, page_bytes = 0;

	static uint64_t Fnv1a64(const void* data, size_t len) {
		const uint8_t* p = (const uint8_t*)data;
		uint64_t h = 14695981039346656037ull;
		for (size_t i = 0; i < len; ++i) {
			h ^= p[i];
			h *= 1099511628211ull;
		}
		return h;
	}
	int by_name(const char* name) const {
		for (size_t i = 0; i < entries.size(); ++i)
			if (entries[i].name == name) return (int)i;
		return -1;
	}
	int by_hash(uint64_t h) const {
		for (size_t i = 0; i < entries.size(); ++i)
			if (entries[i].name_hash == h) return (int)i;
		return -1;
	}
	// binary search of state's row (schema_masks.h:118-139)
	bool transition(const SchemaEntry& e, uint32_t state, uint32_t token, uint32_t* next) const {
		uint32_t lo = rd32(e.offsets_off + (uint64_t)state * 4), hi = rd32(e.offsets_off + (uint64_t)(state + 1) * 4);
		while (lo < hi) {
			const uint32_t mid = lo + (hi - lo) / 2;
			const uint32_t tid = rd32(e.transitions_off + (uint64_t)mid * 8);
			if (tid == token) {
				if (next) *next = rd32(e.transitions_off + (uint64_t)mid * 8 + 4);
				return true;
			}
			if (tid < token) lo = mid + 1; else hi = mid;
		}
		return false;
	}
	const uint8_t* pages(const SchemaEntry& e) const { return bytes.data() + e.pages_off; }

	// false on any malformation (the caller rejects the artifact)
	bool parse(const uint8_t* data, uint64_t size, uint32_t config_vocab) {
		bytes.assign(data, data + size);
		entries.clear();
		const uint8_t* d0 = bytes.data();
		auto r32 = [&](uint64_t off) { uint32_t v; memcpy(&v, d0 + off, 4); return v; };
		auto r64 = [&](uint64_t off) { uint64_t v; memcpy(&v, d0 + off, 8); return v; };
		if (size < 24 || memcmp(d0, "SCM1", 4) != 0 || r32(4) != 1) return false;
		const uint32_t count = r32(8), name_len = r32(16);
		vocab = r32(12);
		if (r32(20) != 0 || count == 0 || count > 65536 || vocab == 0 || vocab != config_vocab) return false;
		const uint64_t manifest_end = 24 + (uint64_t)count * 56 + name_len;
		if (manifest_end > size) return false;
		const uint64_t name_blob = manifest_end - name_len;
		page_bytes = (uint32_t)(((uint64_t)vocab + 7) / 8);
		struct Span { uint64_t off, len; };
		std::vector<Span> occupied;
		auto overlaps = [](const Span& a, const Span& b) { return a.off < b.off + b.len && b.off < a.off + a.len; };
		size_t page_cursor = 0;
		for (uint32_t i = 0; i < count; ++i) {
			const uint64_t d = 24 + (uint64_t)i * 56;
			const uint32_t noff = r32(d), nlen = r32(d + 4);
			SchemaEntry e;
			e.states = r32(d + 8); e.accepting = r32(d + 12); e.transitions = r32(d + 16);
			if (r32(d + 20) != 0) return false;
			e.pages_off = r64(d + 24); e.offsets_off = r64(d + 32); e.accepting_off = r64(d + 40); e.transitions_off = r64(d + 48);
			if (nlen == 0 || (uint64_t)noff + nlen > name_len) return false;
			e.name.assign((const char*)d0 + name_blob + noff, nlen);
			for (const SchemaEntry& o : entries)
				if (o.name == e.name) return false;
			if (e.states == 0 || e.states > 1048576 || e.accepting > e.states || e.transitions > 16777216) return false;
			const Span blocks[4] = {{e.pages_off, (uint64_t)e.states * page_bytes}, {e.offsets_off, ((uint64_t)e.states + 1) * 4},
			                        {e.accepting_off, (uint64_t)e.accepting * 4}, {e.transitions_off, (uint64_t)e.transitions * 8}};
			for (const Span& b : blocks)
				if (b.off < manifest_end || b.off > size || b.len > size - b.off) return false;
			for (const Span& b : blocks)
				for (const Span& p : occupied)
					if (overlaps(b, p)) return false;
			for (int a = 0; a < 4; ++a)
				for (int b = a + 1; b < 4; ++b)
					if (overlaps(blocks[a], blocks[b])) return false;
			for (const Span& b : blocks) occupied.push_back(b);
			if (r32(e.offsets_off) != 0 || r32(e.offsets_off + (uint64_t)e.states * 4) != e.transitions) return false;
			for (uint32_t s = 0; s < e.states; ++s)
				if (r32(e.offsets_off + (uint64_t)s * 4) > r32(e.offsets_off + (uint64_t)(s + 1) * 4)) return false;
			uint32_t prev = 0;
			for (uint32_t a = 0; a < e.accepting; ++a) {
				const uint32_t v = r32(e.accepting_off + (uint64_t)a * 4);
				if (v >= e.states || (a > 0 && v <= prev)) return false;
				prev = v;
			}
			for (uint32_t s = 0; s < e.states; ++s) {
				const uint32_t b0 = r32(e.offsets_off + (uint64_t)s * 4), b1 = r32(e.offsets_off + (uint64_t)(s + 1) * 4);
				uint32_t prev_tok = 0;
				for (uint32_t k = b0; k < b1; ++k) {
					const uint32_t tok = r32(e.transitions_off + (uint64_t)k * 8), nxt = r32(e.transitions_off + (uint64_t)k * 8 + 4);
					if (tok >= vocab || nxt >= e.states || (k > b0 && tok <= prev_tok)) return false;
					prev_tok = tok;
				}
				// a state's mask page has exactly the bits of its row's tokens
				const uint8_t* page = d0 + e.pages_off + (uint64_t)s * page_bytes;
				uint32_t cursor = b0;
				for (uint32_t t = 0; t < vocab; ++t) {
					const bool bit = (page[t >> 3] >> (t & 7)) & 1u;
					bool in_row = false;
					if (cursor < b1 && r32(e.transitions_off + (uint64_t)cursor * 8) == t) {
						in_row = true;
						++cursor;
					}
					if (bit != in_row) return false;
				}
			}
			e.name_hash = Fnv1a64(e.name.data(), e.name.size());
			e.device_page0 = page_cursor;
			page_cursor += e.states;
			entries.push_back(std::move(e));
		}
		return true;
	}
	size_t total_pages() const {
		size_t n = 0;
		for (const SchemaEntry& e : entries) n += e.states;
		return n;
	}

private:
	uint32_t rd32(uint64_t off) const { uint32_t v; memcpy(&v, bytes.data() + off, 4); return v; }
};

}  // namespace sslm
