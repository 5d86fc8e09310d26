// The decode loop on the host, in C++: one call runs up to `max_steps` one-token steps of a
// fixed batch without returning to Python. Per step it writes the step's tokens and
// positions into a pinned buffer, sends them with one copy, launches the captured step graph,
// launches the sampling kernel on the logits, copies the chosen tokens back and waits for
// them; it stops early when a sequence produces a stop token. It allocates nothing: every
// buffer (device and pinned host) is made by the caller and lives as long as the loop.
//
// The reference's loop is the same shape, one sequence at a time: feed the last token, run
// the resident engine, read one token id back (src/main.rs:3760-3883;
// src/inference.rs:2656-2689). The draw of a stochastic step is the reference's stream:
// splitmix64(seed + (position + 1) * golden), top 24 bits (src/inference.rs:6160-6180),
// position being the length of the request's history.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

extern "C" int cml_argmax_rows(const float* logits, int ld, int rows, int vocab, int* out, int* err,
                               unsigned long long* scratch, void* stream);
extern "C" int cml_sample_rows(const float* logits, int ld, int rows, int vocab, float temperature, int top_k,
                               float top_p, float min_p, const float* params_dev, const float* draws, int* out, int* err,
                               void* stream);

struct CmlDecodeLoop {
    int n;                    // sequences of the batch
    int off_tokens, off_row_pos, off_seq_slot, off_seq_start, head_ints;   // places in the step's integer buffer
    int* meta_dev;
    int* meta_host;           // pinned, head_ints ints
    const float* logits;      // [n, ld] written by the graph
    int ld, vocab;
    int* tokens_dev;          // [n] written by the sampling kernel
    int* tokens_host;         // pinned [n]
    int* err_dev;
    unsigned long long* argmax_scratch;
    float* draws_dev;         // [n]
    float* draws_host;        // pinned [n]
};

static uint64_t splitmix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static float unit_draw(uint64_t seed, uint64_t position) {
    const uint64_t state = seed + (position + 1) * 0x9E3779B97F4A7C15ull;
    return (float)(splitmix64(state) >> 40) / (float)(1u << 24);
}

// Fills `loop` (caller-owned, at least cml_decode_loop_size() bytes).
extern "C" int cml_decode_loop_size() { return (int)sizeof(CmlDecodeLoop); }

extern "C" int cml_decode_loop_init(void* loop, int n, int off_tokens, int off_row_pos, int off_seq_slot, int off_seq_start,
                                    int head_ints,
                                    void* meta_dev, void* meta_host, const void* logits, int ld, int vocab,
                                    void* tokens_dev, void* tokens_host, void* err_dev, void* argmax_scratch,
                                    void* draws_dev, void* draws_host) {
    if (!loop || n <= 0 || head_ints <= 0) return -3;
    CmlDecodeLoop* L = (CmlDecodeLoop*)loop;
    L->n = n;
    L->off_tokens = off_tokens; L->off_row_pos = off_row_pos; L->off_seq_slot = off_seq_slot;
    L->off_seq_start = off_seq_start; L->head_ints = head_ints;
    L->meta_dev = (int*)meta_dev; L->meta_host = (int*)meta_host;
    L->logits = (const float*)logits; L->ld = ld; L->vocab = vocab;
    L->tokens_dev = (int*)tokens_dev; L->tokens_host = (int*)tokens_host;
    L->err_dev = (int*)err_dev; L->argmax_scratch = (unsigned long long*)argmax_scratch;
    L->draws_dev = (float*)draws_dev; L->draws_host = (float*)draws_host;
    return 0;
}

// tokens: the token each sequence feeds first; positions: its length now (the place of that token);
// slots: the cache slot of each sequence (the head of the buffer that is sent every step holds them,
// so they are written here and not taken from an earlier batch of the same size).
// history_lens: tokens of each request so far, prompt included (the stream position of its next draw).
// out_tokens: [max_steps][n] chosen tokens; *steps_done: steps run. Stops after the step in which a
// sequence chose one of stop_ids. temperature 0: greedy. Returns 0 or a CUDA error code.
// The block tables in the device buffer must already cover positions[i] + max_steps - 1.
extern "C" int cml_decode_loop_run(void* loop, void* graph_exec, void* stream, const int* tokens, const int* positions,
                                   const int* slots, const int* history_lens, int max_steps, const int* stop_ids, int n_stop,
                                   float temperature, int top_k, float top_p, float min_p, unsigned long long seed,
                                   int* out_tokens, int* steps_done) {
    CmlDecodeLoop* L = (CmlDecodeLoop*)loop;
    cudaStream_t s = (cudaStream_t)stream;
    cudaGraphExec_t exec = (cudaGraphExec_t)graph_exec;
    const int n = L->n;
    *steps_done = 0;
    for (int i = 0; i < n; ++i) {
        L->meta_host[L->off_tokens + i] = tokens[i];
        L->meta_host[L->off_row_pos + i] = positions[i];
        L->meta_host[L->off_seq_slot + i] = slots[i];
        L->meta_host[L->off_seq_start + i] = positions[i];
    }
    for (int step = 0; step < max_steps; ++step) {
        cudaError_t e = cudaMemcpyAsync(L->meta_dev, L->meta_host, (size_t)L->head_ints * sizeof(int),
                                        cudaMemcpyHostToDevice, s);
        if (e != cudaSuccess) return (int)e;
        e = cudaGraphLaunch(exec, s);
        if (e != cudaSuccess) return (int)e;
        int rc;
        if (temperature > 0.f) {
            for (int i = 0; i < n; ++i) L->draws_host[i] = unit_draw(seed, (uint64_t)(history_lens[i] + step));
            e = cudaMemcpyAsync(L->draws_dev, L->draws_host, (size_t)n * sizeof(float), cudaMemcpyHostToDevice, s);
            if (e != cudaSuccess) return (int)e;
            rc = cml_sample_rows(L->logits, L->ld, n, L->vocab, temperature, top_k, top_p, min_p, nullptr, L->draws_dev,
                                 L->tokens_dev, L->err_dev, s);
        } else {
            rc = cml_argmax_rows(L->logits, L->ld, n, L->vocab, L->tokens_dev, L->err_dev, L->argmax_scratch, s);
        }
        if (rc) return rc;
        e = cudaMemcpyAsync(L->tokens_host, L->tokens_dev, (size_t)n * sizeof(int), cudaMemcpyDeviceToHost, s);
        if (e != cudaSuccess) return (int)e;
        e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) return (int)e;
        bool stop = false;
        for (int i = 0; i < n; ++i) {
            const int t = L->tokens_host[i];
            out_tokens[(size_t)step * n + i] = t;
            for (int j = 0; j < n_stop; ++j) stop = stop || (t == stop_ids[j]);
            // the next step feeds this token one position further
            L->meta_host[L->off_tokens + i] = t;
            L->meta_host[L->off_row_pos + i] += 1;
            L->meta_host[L->off_seq_start + i] += 1;
        }
        *steps_done = step + 1;
        if (stop) break;
    }
    return 0;
}

// The loop for greedy requests when the captured graph itself picks each row's token and writes
// it where the next step reads its tokens (the step's integer buffer starts with the tokens).
// Nothing has to come back before the next step can start, so all `steps` steps are queued at
// once: per step one pinned->device copy of that step's positions, the graph, and one
// device->pinned copy of the tokens it chose; the host waits once, at the end.
//   meta_ring: pinned [steps or more][head_ints], every row pre-filled with the arrays that never
//              change (the row -> sequence map); this call writes tokens (row 0), positions and slots.
//   out_tokens: pinned [steps][n].
extern "C" int cml_decode_fed_run(int n, int off_tokens, int off_row_pos, int off_seq_slot, int off_seq_start,
                                  int head_ints, void* meta_dev, int* meta_ring, void* graph_exec, void* stream,
                                  const int* tokens, const int* positions, const int* slots, int steps,
                                  int* out_tokens) {
    if (n <= 0 || steps <= 0 || head_ints < n || off_tokens != 0) return -3;
    cudaStream_t s = (cudaStream_t)stream;
    cudaGraphExec_t exec = (cudaGraphExec_t)graph_exec;
    int* dev = (int*)meta_dev;
    for (int step = 0; step < steps; ++step) {
        int* row = meta_ring + (size_t)step * head_ints;
        for (int i = 0; i < n; ++i) {
            if (step == 0) row[off_tokens + i] = tokens[i];
            row[off_row_pos + i] = positions[i] + step;
            row[off_seq_slot + i] = slots[i];
            row[off_seq_start + i] = positions[i] + step;
        }
        // the first step brings its tokens; later ones leave the device's own choice in place
        const int skip = step == 0 ? 0 : n;
        cudaError_t e = cudaMemcpyAsync(dev + skip, row + skip, (size_t)(head_ints - skip) * sizeof(int),
                                        cudaMemcpyHostToDevice, s);
        if (e != cudaSuccess) return (int)e;
        e = cudaGraphLaunch(exec, s);
        if (e != cudaSuccess) return (int)e;
        e = cudaMemcpyAsync(out_tokens + (size_t)step * n, dev + off_tokens, (size_t)n * sizeof(int),
                            cudaMemcpyDeviceToHost, s);
        if (e != cudaSuccess) return (int)e;
    }
    return (int)cudaStreamSynchronize(s);
}
