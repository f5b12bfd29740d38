// Host-side reader of the `.sslm` v2 container, as far as the forward pass needs it:
// header + integrity hash, section table, CFG1, SIL1, tensor manifests (WGT1/WSC1/ROP1/
// BIA1/DFS1/UFS1), KVC1 keyed constants and the ADP1 adapter prefix, with the load-time
// value gates of the reference (src/model.cpp:945-1407) for the sections read here.
// Layout per docs/sslm_format.md:47-77, :200-238, :242-288, :292-327, :340-365 of the
// reference project. A view borrows the caller's bytes; nothing is copied.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <string_view>
#include <unordered_map>
#include <vector>

namespace sslm {

struct TensorView {
	const uint8_t* data = nullptr;
	uint32_t rank = 0;
	uint32_t shape[4] = {0, 0, 0, 0};
	uint64_t elem_count = 0;
};

struct ConstEntry {
	int64_t v[3] = {0, 0, 0};
	uint32_t words = 0;
};

struct ConfigView {
	uint32_t hidden = 0, layers = 0, heads = 0, kv_heads = 0, head_dim = 0, inter = 0, vocab = 0,
	         context_cap = 0, tie = 0, kv_precision = 0, kv_block = 0;
};

enum : uint32_t {
	kSecConfig = 0, kSecProvenance = 1, kSecWeights = 2, kSecBiases = 3, kSecRope = 4,
	kSecWeightScales = 6, kSecComposition = 7, kSecKvScales = 8, kSecKvRecip = 9,
	kSecSigmoidLut = 12, kSecSchemaMasks = 30, kSecDeltaFold = 40, kSecUFold = 41,
};

class ArtifactView {
public:
	// false + *err on any structural or value-gate rejection
	bool Open(const uint8_t* data, size_t size, std::string* err);

	const ConfigView& config() const { return cfg_; }
	uint32_t flags() const { return flags_; }
	const uint8_t* integrity_hash() const { return data_ + 32; }  // the stored 32 bytes
	bool has(uint32_t section_type) const { return sections_.count(section_type) != 0; }
	const uint8_t* section_data(uint32_t t, uint64_t* size) const;

	const TensorView* weight(const std::string& n) const { return find(weights_, n); }
	const TensorView* weight_scale(const std::string& n) const { return find(wsc_, n); }
	const TensorView* rope(const std::string& n) const { return find(rope_, n); }
	const TensorView* bias(const std::string& n) const { return find(bias_, n); }
	const TensorView* delta_fold(const std::string& n) const { return find(dfs_, n); }
	const TensorView* u_fold(const std::string& n) const { return find(ufs_, n); }
	const std::unordered_map<std::string, TensorView>& delta_folds() const { return dfs_; }
	const ConstEntry* composition(const std::string& n) const { return findc(comp_, n); }
	const ConstEntry* kv_recip(const std::string& n) const { return findc(recip_, n); }
	const int32_t* silu_table() const { return silu_.data(); }

private:
	struct Sec { uint32_t dtype; uint64_t off, size, count; };
	using TMap = std::unordered_map<std::string, TensorView>;
	using CMap = std::unordered_map<std::string, ConstEntry>;
	static const TensorView* find(const TMap& m, const std::string& n) {
		auto it = m.find(n);
		return it == m.end() ? nullptr : &it->second;
	}
	static const ConstEntry* findc(const CMap& m, const std::string& n) {
		auto it = m.find(n);
		return it == m.end() ? nullptr : &it->second;
	}
	bool ParseManifest(uint32_t type, const char magic[4], uint32_t elem_size, TMap& out, std::string* err);
	bool ParseConstants(uint32_t type, uint32_t words, CMap& out, std::string* err);
	bool ValueGates(std::string* err);

	const uint8_t* data_ = nullptr;
	size_t size_ = 0;
	uint32_t flags_ = 0;
	std::unordered_map<uint32_t, Sec> sections_;
	ConfigView cfg_;
	TMap weights_, wsc_, rope_, bias_, dfs_, ufs_;
	CMap comp_, kvscale_, recip_;
	std::vector<int32_t> silu_;
};

void Sha256(const uint8_t* data, size_t size, const uint8_t* zero_from, size_t zero_len, uint8_t out[32]);

}  // namespace sslm
