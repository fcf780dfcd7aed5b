// Drives include/nvk_b200_host.hpp from a C++ host: reads operands the Python test wrote into a
// directory, runs a linear (plain, residual update, norm in front), an MLP and a grouped MoE decode step
// through the host layer, and writes the results back for the test to compare with the oracle.  Linked
// against the host emulation of the library in the CPU suite; the same source links against
// libnvk_b200.so on a GPU box (buffers then come from cudaMalloc instead of emu_alloc).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <string>
#include <vector>

#include "nvk_b200_host.hpp"

extern "C" void* emu_alloc(size_t bytes, int front);
extern "C" void emu_free(void* p);
extern "C" void emu_install_fault_handler(void);

namespace {

std::string g_dir;

std::vector<char> read_file(const std::string& name) {
    std::ifstream f(g_dir + "/" + name, std::ios::binary);
    if (!f) {
        std::fprintf(stderr, "missing %s\n", name.c_str());
        std::exit(2);
    }
    return std::vector<char>((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
}

// a "device" buffer holding the file's bytes
template <class T>
T* upload(const std::string& name) {
    const std::vector<char> h = read_file(name);
    void* d = emu_alloc(h.size() ? h.size() : 1, 0);
    std::memcpy(d, h.data(), h.size());
    return static_cast<T*>(d);
}

template <class T>
T* device_zeros(size_t count) {
    void* d = emu_alloc(count ? count * sizeof(T) : 1, 0);
    std::memset(d, 0, count * sizeof(T));
    return static_cast<T*>(d);
}

template <class T>
void download(const std::string& name, const T* d, size_t count) {
    std::ofstream f(g_dir + "/" + name, std::ios::binary);
    f.write(reinterpret_cast<const char*>(d), (std::streamsize)(count * sizeof(T)));
}

std::map<std::string, double> read_meta() {
    std::map<std::string, double> m;
    std::ifstream f(g_dir + "/meta.txt");
    std::string key;
    double v;
    while (f >> key >> v) m[key] = v;
    return m;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc < 2) return 2;
    g_dir = argv[1];
    emu_install_fault_handler();   // an access outside a buffer ends the run with a message
    using namespace nvk::host;
    auto meta = read_meta();
    void* stream = nullptr;
    try {
        // ---- one linear: plain, residual update, RMSNorm in front ----
        {
            const int m = (int)meta["lin_m"], n = (int)meta["lin_n"], k = (int)meta["lin_k"];
            Nvfp4Linear lin(upload<uint8_t>("lin_packed.bin"), upload<uint8_t>("lin_scales.bin"), (float)meta["lin_alpha"], k, n);
            const uint16_t* x = upload<uint16_t>("lin_x.bin");
            uint16_t* y = device_zeros<uint16_t>((size_t)m * n);
            lin.forward_into(stream, x, y, m);
            download("out_lin.bin", y, (size_t)m * n);
            lin.forward_into(stream, x, y, 1);                         // the M = 1 route on the first row
            download("out_lin_m1.bin", y, (size_t)n);
            uint16_t* h = upload<uint16_t>("lin_residual.bin");
            lin.forward_residual_into(stream, x, nullptr, h, h, m);    // in place
            download("out_lin_residual.bin", h, (size_t)m * n);
            const uint16_t* nw = upload<uint16_t>("lin_norm_w.bin");
            uint16_t* scratch = device_zeros<uint16_t>((size_t)m * k);
            lin.forward_prenorm_decode_into(stream, x, nw, (float)meta["eps"], y, m, scratch);
            download("out_lin_prenorm.bin", y, (size_t)m * n);
            lin.forward_prenorm_decode_into(stream, x, nw, (float)meta["eps"], y, m > 8 ? 8 : m, nullptr);
            download("out_lin_prenorm_few.bin", y, (size_t)(m > 8 ? 8 : m) * n);
        }
        // ---- MLP ----
        {
            const int m = (int)meta["mlp_m"], hidden = (int)meta["mlp_hidden"], inter = (int)meta["mlp_inter"];
            Nvfp4Linear gate(upload<uint8_t>("mlp_gate_packed.bin"), upload<uint8_t>("mlp_gate_scales.bin"), (float)meta["mlp_gate_alpha"], hidden, inter);
            Nvfp4Linear up(upload<uint8_t>("mlp_up_packed.bin"), upload<uint8_t>("mlp_up_scales.bin"), (float)meta["mlp_up_alpha"], hidden, inter);
            Nvfp4Linear down(upload<uint8_t>("mlp_down_packed.bin"), upload<uint8_t>("mlp_down_scales.bin"), (float)meta["mlp_down_alpha"], inter, hidden);
            Nvfp4Mlp mlp(gate, up, down);
            const uint16_t* x = upload<uint16_t>("mlp_x.bin");
            uint16_t* g = device_zeros<uint16_t>((size_t)m * inter);
            uint16_t* u = device_zeros<uint16_t>((size_t)m * inter);
            uint16_t* y = device_zeros<uint16_t>((size_t)m * hidden);
            mlp.forward_into(stream, x, g, u, y, m);
            download("out_mlp.bin", y, (size_t)m * hidden);
        }
        // ---- grouped MoE decode step ----
        {
            const int n = (int)meta["moe_n"], E = (int)meta["moe_E"], k = (int)meta["moe_topk"];
            const int hidden = (int)meta["moe_hidden"], inter = (int)meta["moe_inter"];
            MoeGroupedWeights w;
            w.gate = {upload<uint8_t>("moe_gate_packed.bin"), upload<uint8_t>("moe_gate_scales.bin"), upload<float>("moe_gate_alphas.bin")};
            w.up = {upload<uint8_t>("moe_up_packed.bin"), upload<uint8_t>("moe_up_scales.bin"), upload<float>("moe_up_alphas.bin")};
            w.down = {upload<uint8_t>("moe_down_packed.bin"), upload<uint8_t>("moe_down_scales.bin"), upload<float>("moe_down_alphas.bin")};
            w.hidden = hidden; w.inter = inter; w.num_experts = E;
            GroupedDecodeContext c;
            c.max_tokens = n; c.top_k = k;
            const size_t slots = (size_t)n * k;
            c.topk_ids = device_zeros<int32_t>(slots);
            c.topk_weights = device_zeros<float>(slots);
            c.perm_token = device_zeros<int32_t>(slots);
            c.offsets = device_zeros<int32_t>((size_t)E + 1);
            c.inv_perm = device_zeros<int32_t>(slots);
            c.counts = device_zeros<int32_t>((size_t)E);
            c.active = device_zeros<int32_t>(slots < (size_t)E ? slots : (size_t)E);
            c.n_active = device_zeros<int32_t>(1);
            c.status = device_zeros<int32_t>(1);
            c.gate_out = device_zeros<uint16_t>(slots * inter);
            c.up_out = device_zeros<uint16_t>(slots * inter);
            c.down_out = device_zeros<uint16_t>(slots * hidden);
            c.y_acc = device_zeros<float>((size_t)n * hidden);
            forward_grouped_decode(stream, w, c, upload<uint16_t>("moe_x.bin"), upload<float>("moe_logits.bin"), n);
            download("out_moe.bin", c.y_acc, (size_t)n * hidden);
            download("out_moe_ids.bin", c.topk_ids, slots);
            download("out_moe_status.bin", c.status, 1);
        }
        // ---- the fused row-parallel linear with a world of one: the plain linear's bits ----
        {
            const int m = (int)meta["lin_m"] > 8 ? 8 : (int)meta["lin_m"], n = (int)meta["lin_n"], k = (int)meta["lin_k"];
            Nvfp4Linear lin(upload<uint8_t>("lin_packed.bin"), upload<uint8_t>("lin_scales.bin"), (float)meta["lin_alpha"], k, n);
            const int max_ctas = 64, max_rows = 8;
            void* buf = device_zeros<uint8_t>(nvk_b200_tp_fused_buffer_bytes(1, max_ctas, max_rows));
            const void* bufs[1] = {buf};
            PeerExchange px = {bufs, 0, 1, max_ctas, max_rows, device_zeros<uint32_t>(max_ctas), device_zeros<int>(1)};
            uint16_t* y = device_zeros<uint16_t>((size_t)m * n);
            const bool ran = tp_linear_allreduce(stream, px, lin, upload<uint16_t>("lin_x.bin"), nullptr, nullptr, y, m);
            std::printf("tp fused: %d err %d\n", ran ? 1 : 0, *px.err);
            download("out_lin_tp1.bin", y, (size_t)m * n);
        }
        // ---- a refusal arrives as an exception that names the entry point ----
        {
            Nvfp4Linear lin(reinterpret_cast<const uint8_t*>(0x1000), reinterpret_cast<const uint8_t*>(0x1000), 1.f, 144, 128);
            try {
                lin.forward_residual_into(stream, reinterpret_cast<const uint16_t*>(0x1000), nullptr,
                                          reinterpret_cast<const uint16_t*>(0x1000), reinterpret_cast<uint16_t*>(0x1000), 4);
                std::printf("residual refusal: none\n");
            } catch (const Error& e) {
                std::printf("residual refusal: %s %d\n", e.entry.c_str(), e.status);
            }
        }
    } catch (const std::exception& e) {
        std::fprintf(stderr, "host_check: %s\n", e.what());
        return 1;
    }
    std::printf("host_check ok\n");
    return 0;
}
