// End-to-end LSTM cell step through the C++ front end, the call a user of the reference makes: host arrays in,
// lazy Array / op:: expression, evaluation, host arrays out, every step (benchmark configuration 2: fp32, B x H,
// weights [H, 4H], gate blocks i | f | o | g).  bench.py runs it for its end-to-end figure.
//
//   lstm_cell_e2e <gpu> <B> <H> <warmup> <steps>   ->   one JSON line with ms_per_step and a checksum
//
// Inputs live in page-locked buffers (dalib200_host_alloc) that the step borrows, results are read straight into
// page-locked buffers; the weights are Arrays that stay on the device, as in a recurrent loop.
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "dali/array/array.h"
#include "dali/array/op.h"
#include "dali_b200.h"

static float* pinned(size_t n) {
    void* p = nullptr;
    if (dalib200_host_alloc(n * sizeof(float), &p) != 0) { std::fprintf(stderr, "dalib200_host_alloc failed\n"); std::exit(2); }
    return static_cast<float*>(p);
}

int main(int argc, char** argv) {
    if (argc < 6) { std::fprintf(stderr, "usage: lstm_cell_e2e <gpu> <B> <H> <warmup> <steps>\n"); return 2; }
    const int gpu = std::atoi(argv[1]), B = std::atoi(argv[2]), H = std::atoi(argv[3]);
    const int warmup = std::atoi(argv[4]), steps = std::atoi(argv[5]);
    try {
        if (dalib200_init(0) != 0) { std::fprintf(stderr, "no CUDA device\n"); return 2; }
        memory::default_preferred_device = memory::Device::gpu(gpu);
        std::mt19937 gen(1234 + 1 + gpu);
        std::normal_distribution<float> n01(0.0f, 1.0f);
        float *x = pinned((size_t)B * H), *h = pinned((size_t)B * H), *c = pinned((size_t)B * H);
        float *h_out = pinned((size_t)B * H), *c_out = pinned((size_t)B * H);
        for (size_t i = 0; i < (size_t)B * H; ++i) { x[i] = n01(gen); h[i] = n01(gen); c[i] = n01(gen); }
        Array Wx({H, 4 * H}, DTYPE_FLOAT), Wh({H, 4 * H}, DTYPE_FLOAT), b = Array::zeros({4 * H}, DTYPE_FLOAT);
        {
            std::vector<float> w((size_t)H * 4 * H);
            for (Array* W : {&Wx, &Wh}) {
                for (float& v : w) v = 0.02f * n01(gen);
                W->assign(Array::borrow_host(w.data(), {H, 4 * H}, DTYPE_FLOAT));
                W->eval();
            }
            b.eval();
        }
        auto step = [&]() {
            Array X = Array::borrow_host(x, {B, H}, DTYPE_FLOAT), Hh = Array::borrow_host(h, {B, H}, DTYPE_FLOAT);
            Array C = Array::borrow_host(c, {B, H}, DTYPE_FLOAT);
            Array gates = op::dot(X, Wx) + op::dot(Hh, Wh) + b[Broadcast()];
            Array i = op::sigmoid(gates[Slice()][Slice(0, H)]), f = op::sigmoid(gates[Slice()][Slice(H, 2 * H)]);
            Array o = op::sigmoid(gates[Slice()][Slice(2 * H, 3 * H)]), g = op::tanh(gates[Slice()][Slice(3 * H, 4 * H)]);
            Array c_new = f * C + i * g;
            Array h_new = o * op::tanh(c_new);
            Array::eval_together({c_new, h_new}, /*wait=*/false);
            h_new.to_host(h_out, /*wait=*/false);      // both copies queued behind the kernels, one synchronisation
            c_new.to_host(c_out);
        };
        for (int i = 0; i < warmup; ++i) step();
        const auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < steps; ++i) step();
        const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / (steps > 0 ? steps : 1);
        double sum = 0;
        for (size_t i = 0; i < (size_t)B * H; ++i) sum += (double)h_out[i] + (double)c_out[i];
        std::printf("{\"ms_per_step\": %.6f, \"steps\": %d, \"checksum\": %.9g, \"h2d_bytes_per_step\": %zu, \"d2h_bytes_per_step\": %zu}\n", ms,
                    steps, sum, (size_t)3 * B * H * 4, (size_t)2 * B * H * 4);
    } catch (const std::exception& e) {
        std::fprintf(stderr, "lstm_cell_e2e: %s\n", e.what());
        return 1;
    }
    return 0;
}
