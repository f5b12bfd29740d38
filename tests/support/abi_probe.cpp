// A caller written against the REFERENCE's own header (include/superslm/sslm_abi.h of the
// reference tree, given on the compiler's include path) and linked against libsslm_b200.so:
// the drop-in boundary exercised from C++ exactly as a program built for the reference would
// use it -- map, pool, workspace, sequence, chunked prefill, sliced greedy decode, save.
// Prints the decoded tokens and an FNV-1a digest of the save blob, which the test compares with
// the reference library's record for the same artifact and prompt. Test infrastructure.
//
//   abi_probe <artifact.sslm> <prompt.i32> <chunk_budget> <layer_budget> <decode_tokens>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "superslm/sslm_abi.h"

static std::vector<uint8_t> read_file(const char* path) {
	std::vector<uint8_t> out;
	FILE* f = fopen(path, "rb");
	if (!f) return out;
	fseek(f, 0, SEEK_END);
	const long n = ftell(f);
	fseek(f, 0, SEEK_SET);
	out.resize((size_t)n);
	if (n > 0 && fread(out.data(), 1, (size_t)n, f) != (size_t)n) out.clear();
	fclose(f);
	return out;
}
static void* aligned(std::vector<uint8_t>& store, size_t bytes) {
	store.assign(bytes + SSLM_ABI_ALIGNMENT_BYTES, 0);
	const uintptr_t a = (uintptr_t)store.data();
	return (void*)((a + SSLM_ABI_ALIGNMENT_BYTES - 1) / SSLM_ABI_ALIGNMENT_BYTES * SSLM_ABI_ALIGNMENT_BYTES);
}
#define CHECK(call)                                                         \
	do {                                                                    \
		const sslm_status st_ = (call);                                     \
		if (st_ != SSLM_OK) {                                               \
			printf("FAIL %s -> %d\n", #call, (int)st_);                     \
			return 2;                                                       \
		}                                                                   \
	} while (0)

int main(int argc, char** argv) {
	if (argc != 6) return 1;
	const std::vector<uint8_t> art = read_file(argv[1]);
	const std::vector<uint8_t> praw = read_file(argv[2]);
	const int32_t chunk = atoi(argv[3]), budget = atoi(argv[4]), ndec = atoi(argv[5]);
	if (art.empty() || praw.empty()) return 1;
	const int32_t* prompt = (const int32_t*)praw.data();
	const int32_t count = (int32_t)(praw.size() / 4);

	sslm_model model = nullptr;
	CHECK(sslm_model_map(art.data(), art.size(), &model));
	const size_t pool_bytes = sslm_kv_block_size(model) + sslm_kv_pool_overhead_size(model, 1);
	std::vector<uint8_t> pool_store, ws_store;
	sslm_kv_pool pool = nullptr;
	CHECK(sslm_kv_pool_create(model, aligned(pool_store, pool_bytes), pool_bytes, 1, &pool));
	sslm_config cfg = {1, chunk, budget, 0};
	const size_t ws_bytes = sslm_workspace_size(model, &cfg);
	sslm_workspace ws = nullptr;
	CHECK(sslm_workspace_create(model, &cfg, aligned(ws_store, ws_bytes), ws_bytes, &ws));
	sslm_seq seq = nullptr;
	CHECK(sslm_seq_create(model, &pool, &seq));

	int32_t done = 0;
	while (done < count) {
		int32_t consumed = 0;
		CHECK(sslm_prefill(model, seq, prompt + done, count - done, chunk, SSLM_SPAN_PROMPT, ws, &consumed));
		if (consumed <= 0) return 3;
		done += consumed;
	}
	sslm_decode_params params = {};
	params.layer_budget = budget;
	printf("tokens");
	for (int produced = 0; produced < ndec;) {
		int32_t tok = -1;
		CHECK(sslm_decode_step(model, &seq, 1, &params, ws, &tok));
		if (tok >= 0) {
			printf(" %d", tok);
			++produced;
		}
	}
	printf("\n");
	size_t n = 0;
	sslm_seq_save(seq, nullptr, &n);
	std::vector<uint8_t> blob(n);
	CHECK(sslm_seq_save(seq, blob.data(), &n));
	uint64_t h = 1469598103934665603ull;
	for (size_t i = 0; i < n; ++i) h = (h ^ blob[i]) * 1099511628211ull;
	printf("blob %zu %016llx\n", n, (unsigned long long)h);
	CHECK(sslm_seq_release(seq));
	CHECK(sslm_workspace_destroy(ws));
	CHECK(sslm_kv_pool_destroy(pool));
	CHECK(sslm_model_unmap(model));
	return 0;
}
