#include "sslm_artifact.h"

#include <cstring>

namespace sslm {

namespace {
inline uint32_t rd32(const uint8_t* p) {
	return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}
inline uint64_t rd64(const uint8_t* p) { return (uint64_t)rd32(p) | ((uint64_t)rd32(p + 4) << 32); }

bool fail(std::string* err, const std::string& m) {
	if (err) *err = m;
	return false;
}

// FIPS 180-4 SHA-256, streaming over 64-byte blocks.
struct Sha {
	uint32_t h[8] = {0x6a09e667u, 0xbb67ae85u, 0x3c6ef372u, 0xa54ff53au,
	                 0x510e527fu, 0x9b05688cu, 0x1f83d9abu, 0x5be0cd19u};
	uint8_t buf[64];
	size_t fill = 0;
	uint64_t total = 0;
	static uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
	void block(const uint8_t* p) {
		static const uint32_t k[64] = {
		    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5,
		    0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174,
		    0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
		    0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967,
		    0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
		    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
		    0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
		    0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};
		uint32_t w[64];
		for (int i = 0; i < 16; ++i)
			w[i] = ((uint32_t)p[4 * i] << 24) | ((uint32_t)p[4 * i + 1] << 16) | ((uint32_t)p[4 * i + 2] << 8) | p[4 * i + 3];
		for (int i = 16; i < 64; ++i) {
			uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
			uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
			w[i] = w[i - 16] + s0 + w[i - 7] + s1;
		}
		uint32_t a = h[0], b = h[1], c = h[2], d = h[3], e = h[4], f = h[5], g = h[6], hh = h[7];
		for (int i = 0; i < 64; ++i) {
			uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
			uint32_t ch = (e & f) ^ (~e & g);
			uint32_t t1 = hh + S1 + ch + k[i] + w[i];
			uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
			uint32_t mj = (a & b) ^ (a & c) ^ (b & c);
			uint32_t t2 = S0 + mj;
			hh = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
		}
		h[0] += a; h[1] += b; h[2] += c; h[3] += d; h[4] += e; h[5] += f; h[6] += g; h[7] += hh;
	}
	void update(const uint8_t* p, size_t n) {
		total += n;
		if (fill) {
			size_t t = 64 - fill < n ? 64 - fill : n;
			memcpy(buf + fill, p, t);
			fill += t; p += t; n -= t;
			if (fill == 64) { block(buf); fill = 0; }
		}
		while (n >= 64) { block(p); p += 64; n -= 64; }
		if (n) { memcpy(buf, p, n); fill = n; }
	}
	void finish(uint8_t out[32]) {
		uint64_t bits = total * 8;
		uint8_t pad = 0x80;
		update(&pad, 1);
		uint8_t z = 0;
		while (fill != 56) update(&z, 1);
		uint8_t len[8];
		for (int i = 0; i < 8; ++i) len[i] = (uint8_t)(bits >> (56 - 8 * i));
		update(len, 8);
		for (int i = 0; i < 8; ++i) {
			out[4 * i] = (uint8_t)(h[i] >> 24); out[4 * i + 1] = (uint8_t)(h[i] >> 16);
			out[4 * i + 2] = (uint8_t)(h[i] >> 8); out[4 * i + 3] = (uint8_t)h[i];
		}
	}
};
}  // namespace

void Sha256(const uint8_t* data, size_t size, const uint8_t* zero_from, size_t zero_len, uint8_t out[32]) {
	Sha s;
	if (zero_from && zero_from >= data && zero_from + zero_len <= data + size) {
		s.update(data, (size_t)(zero_from - data));
		std::vector<uint8_t> z(zero_len, 0);
		s.update(z.data(), zero_len);
		s.update(zero_from + zero_len, size - (size_t)(zero_from - data) - zero_len);
	} else {
		s.update(data, size);
	}
	s.finish(out);
}

const uint8_t* ArtifactView::section_data(uint32_t t, uint64_t* size) const {
	auto it = sections_.find(t);
	if (it == sections_.end()) return nullptr;
	if (size) *size = it->second.size;
	return data_ + it->second.off;
}

bool ArtifactView::ParseManifest(uint32_t type, const char magic[4], uint32_t esz, TMap& out, std::string* err) {
	auto it = sections_.find(type);
	if (it == sections_.end()) return true;
	const uint8_t* b = data_ + it->second.off;
	const uint64_t size = it->second.size;
	if (size < 16 || memcmp(b, magic, 4) != 0 || rd32(b + 4) != 1) return fail(err, "bad tensor manifest header");
	const uint32_t n = rd32(b + 8), name_len = rd32(b + 12);
	if (n > 65536) return fail(err, "too many tensors");
	const uint64_t names_off = 16 + (uint64_t)n * 48, floor = names_off + name_len;
	if (floor > size) return fail(err, "manifest out of bounds");
	for (uint32_t i = 0; i < n; ++i) {
		const uint8_t* d = b + 16 + (uint64_t)i * 48;
		const uint32_t no = rd32(d), nl = rd32(d + 4), rank = rd32(d + 8);
		if (nl == 0 || (uint64_t)no + nl > name_len) return fail(err, "bad tensor name");
		if (rank == 0 || rank > 4) return fail(err, "bad tensor rank");
		TensorView t;
		t.rank = rank;
		uint64_t prod = 1;
		for (uint32_t k = 0; k < 4; ++k) {
			t.shape[k] = rd32(d + 12 + 4 * k);
			if (k < rank) {
				if (t.shape[k] == 0) return fail(err, "zero shape entry");
				if (prod > UINT64_MAX / t.shape[k]) return fail(err, "shape overflow");
				prod *= t.shape[k];
			} else if (t.shape[k] != 0) {
				return fail(err, "shape entry past rank");
			}
		}
		const uint64_t off = rd64(d + 28);
		t.elem_count = rd64(d + 36);
		if (t.elem_count != prod || rd32(d + 44) != 0) return fail(err, "bad tensor descriptor");
		if (off % esz != 0 || off < floor || t.elem_count > (size - (off < size ? off : size)) / esz || off > size)
			return fail(err, "tensor out of bounds");
		t.data = b + off;
		std::string name((const char*)b + names_off + no, nl);
		if (!out.emplace(name, t).second) return fail(err, "duplicate tensor name");
	}
	return true;
}

bool ArtifactView::ParseConstants(uint32_t type, uint32_t words, CMap& out, std::string* err) {
	auto it = sections_.find(type);
	if (it == sections_.end()) return true;
	const uint8_t* b = data_ + it->second.off;
	const uint64_t size = it->second.size;
	if (size < 24 || memcmp(b, "KVC1", 4) != 0 || rd32(b + 4) != 1) return fail(err, "bad KVC1 header");
	const uint32_t n = rd32(b + 8), w = rd32(b + 12), name_len = rd32(b + 16);
	if (n > 1048576 || w != words || rd32(b + 20) != 0) return fail(err, "bad KVC1 fields");
	const uint64_t vbase = 24 + (uint64_t)n * 8, nbase = vbase + (uint64_t)n * w * 8;
	if (nbase + name_len > size) return fail(err, "KVC1 out of bounds");
	for (uint32_t i = 0; i < n; ++i) {
		const uint32_t no = rd32(b + 24 + 8 * (uint64_t)i), nl = rd32(b + 24 + 8 * (uint64_t)i + 4);
		if (nl == 0 || (uint64_t)no + nl > name_len) return fail(err, "bad KVC1 name");
		ConstEntry e;
		e.words = w;
		for (uint32_t k = 0; k < w; ++k) e.v[k] = (int64_t)rd64(b + vbase + ((uint64_t)i * w + k) * 8);
		if (!out.emplace(std::string((const char*)b + nbase + no, nl), e).second)
			return fail(err, "duplicate KVC1 name");
	}
	return true;
}

bool ArtifactView::ValueGates(std::string* err) {
	// CompositionConstants: |m| <= 2^31-1, e in [-80, 7] (src/model.cpp:945-966)
	for (auto& kv : comp_) {
		const int64_t m = kv.second.v[0], e = kv.second.v[1];
		if (m < -2147483647ll || m > 2147483647ll || e < -80 || e > 7) return fail(err, "composition constant out of domain: " + kv.first);
	}
	// WeightScales: identity in {0,1}, shift in [0,31] (:976-1015); amplifying folds: exponent in [-31,31] (:380-405)
	for (auto& kv : wsc_) {
		if (kv.second.elem_count % 3) return fail(err, "weight scale triple count");
		for (uint64_t r = 0; r < kv.second.elem_count / 3; ++r) {
			const int32_t id = (int32_t)rd32(kv.second.data + (r * 3) * 4), sh = (int32_t)rd32(kv.second.data + (r * 3 + 2) * 4);
			if (id < 0 || id > 1 || sh < 0 || sh > 31) return fail(err, "weight scale row out of domain: " + kv.first);
		}
	}
	for (const TMap* mp : {&dfs_, &ufs_}) {
		for (auto& kv : *mp) {
			if (kv.second.elem_count % 3) return fail(err, "amplifying fold triple count");
			for (uint64_t r = 0; r < kv.second.elem_count / 3; ++r) {
				const int32_t id = (int32_t)rd32(kv.second.data + (r * 3) * 4), ex = (int32_t)rd32(kv.second.data + (r * 3 + 2) * 4);
				if (id < 0 || id > 1 || ex < -31 || ex > 31) return fail(err, "amplifying fold row out of domain: " + kv.first);
			}
		}
	}
	// RopeTables: |v| <= 2^30 (:1021-1036) and shape join with CFG1 (:1309-1336)
	for (auto& kv : rope_) {
		for (uint64_t i = 0; i < kv.second.elem_count; ++i) {
			const int64_t v = (int64_t)rd64(kv.second.data + 8 * i);
			if (v < -(1ll << 30) || v > (1ll << 30)) return fail(err, "rope entry out of domain");
		}
		if ((kv.first == "cos" || kv.first == "sin") &&
		    kv.second.elem_count != (uint64_t)cfg_.context_cap * (cfg_.head_dim / 2))
			return fail(err, "rope table shape does not match config");
	}
	for (auto& kv : kvscale_) {
		if (kv.second.v[0] < (1ll << 30) || kv.second.v[0] > (1ll << 31) - 1) return fail(err, "kv landing scale out of domain");
	}
	for (auto& kv : recip_) {
		if (kv.second.v[1] < -60 || kv.second.v[2] < (1ll << 31) + 1 || kv.second.v[2] > (1ll << 32))
			return fail(err, "kv landing reciprocal out of domain");
	}
	// geometry join (CheckConfigGeometry, src/model.cpp:1268-1307)
	if (cfg_.kv_heads > cfg_.heads || cfg_.heads % cfg_.kv_heads != 0 ||
	    (uint64_t)cfg_.heads * cfg_.head_dim != cfg_.hidden)
		return fail(err, "config geometry mismatch");
	return true;
}

bool ArtifactView::Open(const uint8_t* data, size_t size, std::string* err) {
	data_ = data;
	size_ = size;
	if (!data || size < 64 || memcmp(data, "SSLM", 4) != 0) return fail(err, "not an .sslm artifact");
	if (rd32(data + 4) != 2 || rd32(data + 8) != 64) return fail(err, "unsupported container version");
	const uint32_t nsec = rd32(data + 12);
	flags_ = rd32(data + 16);
	if (nsec > 4096 || (flags_ & ~0x3u) != 0 || rd32(data + 20) != 0 || rd64(data + 24) != size)
		return fail(err, "bad container header");
	const uint64_t table_end = 64 + (uint64_t)nsec * 40;
	if (table_end > size) return fail(err, "section table out of bounds");
	uint8_t digest[32];
	Sha256(data, size, data + 32, 32, digest);
	if (memcmp(digest, data + 32, 32) != 0) return fail(err, "integrity hash mismatch");
	static const uint32_t kDtSize[7] = {1, 1, 4, 8, 1, 4, 8};
	for (uint32_t i = 0; i < nsec; ++i) {
		const uint8_t* r = data + 64 + (uint64_t)i * 40;
		const uint32_t type = rd32(r), dt = rd32(r + 4), align = rd32(r + 32);
		Sec s{dt, rd64(r + 8), rd64(r + 16), rd64(r + 24)};
		if (dt > 6 || align < 8 || align > 4096 || (align & (align - 1)) || rd32(r + 36) != 0) return fail(err, "bad section row");
		if (s.off < table_end || s.off % align || s.off > size || s.size > size - s.off || s.size != s.count * kDtSize[dt])
			return fail(err, "section out of bounds");
		if (!sections_.emplace(type, s).second) return fail(err, "duplicate section type");
	}
	// CFG1
	{
		auto it = sections_.find(kSecConfig);
		if (it == sections_.end() || it->second.size != 84) return fail(err, "missing or mis-sized Config");
		const uint8_t* c = data + it->second.off;
		if (memcmp(c, "CFG1", 4) != 0 || rd32(c + 4) != 1) return fail(err, "bad CFG1");
		cfg_.hidden = rd32(c + 8); cfg_.layers = rd32(c + 12); cfg_.heads = rd32(c + 16);
		cfg_.kv_heads = rd32(c + 20); cfg_.head_dim = rd32(c + 24); cfg_.inter = rd32(c + 28);
		cfg_.vocab = rd32(c + 32); cfg_.context_cap = rd32(c + 36); cfg_.tie = rd32(c + 40);
		cfg_.kv_precision = rd32(c + 44); cfg_.kv_block = rd32(c + 48);
		if (!cfg_.hidden || !cfg_.layers || !cfg_.heads || !cfg_.kv_heads || !cfg_.head_dim || (cfg_.head_dim & 1) ||
		    !cfg_.inter || !cfg_.vocab || !cfg_.context_cap || cfg_.tie > 1 || cfg_.kv_precision > 1 ||
		    !cfg_.kv_block || rd32(c + 64) != 0)
			return fail(err, "CFG1 field out of domain");
	}
	// SIL1
	{
		auto it = sections_.find(kSecSigmoidLut);
		if (it == sections_.end() || it->second.size != 4116) return fail(err, "missing or mis-sized SigmoidLut");
		const uint8_t* s = data + it->second.off;
		if (memcmp(s, "SIL1", 4) != 0 || rd32(s + 4) != 1 || rd32(s + 8) != 1025 || rd32(s + 12) != 0) return fail(err, "bad SIL1");
		silu_.resize(1025);
		for (int i = 0; i < 1025; ++i) silu_[i] = (int32_t)rd32(s + 16 + 4 * i);
	}
	if (!ParseManifest(kSecWeights, "WGT1", 1, weights_, err)) return false;
	if (!ParseManifest(kSecWeightScales, "WSC1", 4, wsc_, err)) return false;
	if (!ParseManifest(kSecRope, "ROP1", 8, rope_, err)) return false;
	if (!ParseManifest(kSecBiases, "BIA1", 8, bias_, err)) return false;
	if (!ParseManifest(kSecDeltaFold, "DFS1", 4, dfs_, err)) return false;
	if (!ParseManifest(kSecUFold, "UFS1", 4, ufs_, err)) return false;
	if (!ParseConstants(kSecComposition, 2, comp_, err)) return false;
	if (!ParseConstants(kSecKvScales, 2, kvscale_, err)) return false;
	if (!ParseConstants(kSecKvRecip, 3, recip_, err)) return false;
	return ValueGates(err);
}

}  // namespace sslm
