// Exercises the header-only C++ class layer (include/qmlp/*.h) the way a C++ user of the reference library would:
// build a network from a JSON text, query its layout, and (mode "gpu") run inference, forward and adjoint on tensors
// filled from values the Python side of the test wrote to a file. Output: "key value..." lines for the test to parse.
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>
#include <vector>

#include <qmlp/fused_network.h>

using namespace qmlp;

static std::string readFile(const char* path)
{
    std::ifstream in(path, std::ios::binary);
    std::stringstream ss;
    ss << in.rdbuf();
    return ss.str();
}

static std::vector<float> readFloats(const std::string& path)
{
    std::ifstream in(path, std::ios::binary);
    std::vector<char> bytes((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
    std::vector<float> v(bytes.size() / 4);
    std::memcpy(v.data(), bytes.data(), v.size() * 4);
    return v;
}

template <class T>
static void writeRaw(const std::string& path, const std::vector<T>& v)
{
    std::ofstream out(path, std::ios::binary);
    out.write(reinterpret_cast<const char*>(v.data()), static_cast<std::streamsize>(v.size() * sizeof(T)));
}

int main(int argc, char** argv)
{
    if (argc < 3) {
        std::fprintf(stderr, "usage: shim_check layout|gpu <spec.json> [data folder]\n");
        return 2;
    }
    const std::string mode = argv[1];
    const std::string cfg = readFile(argv[2]);
    try {
        QuickMLP::Instance().setLogLevel("error");
        // a specification that cannot be parsed must surface as qmlp::configuration_error
        try {
            FusedNetwork bad("{\"num_inputs\": 3, \"num_outputs\": 1, \"encodings\": [{\"id\": \"NoSuchEncoding\"}], \"network\": []}", ".");
            std::cout << "bad_spec accepted\n";
        } catch (const configuration_error& e) {
            std::cout << "bad_spec configuration_error\n";
        }
        FusedNetwork net(cfg, ".");
        std::cout << "channels " << net.channelsIn() << " " << net.channelsOut() << "\n";
        std::cout << "layers " << net.numLayers() << " encodings " << net.numEncodings() << "\n";
        std::cout << "parameters " << net.networkParameterCount() << " precision "
                  << (net.networkParameterPrecision(Tensor::INFERENCE) == Tensor::HALF ? "half" : "other") << " "
                  << (net.networkParameterPrecision(Tensor::GRADIENTS) == Tensor::FLOAT ? "float" : "other") << "\n";
        for (int i = 0; i < net.numEncodings(); ++i) {
            auto e = net.encoding(i);
            std::cout << "encoding " << i << " " << e->id() << " out " << e->numOutputChannels() << " max_in " << e->maxInputChannel()
                      << " params " << e->parameterCount() << " levels " << e->levels().size() << "\n";
        }
        // views into a (fake) flat parameter vector: offsets and shapes of every layer
        std::vector<char> flat(static_cast<size_t>(net.networkParameterCount()) * 2 + 16);
        for (int l = 0; l < net.numLayers(); ++l) {
            Tensor w = net.networkParameter(l, false, flat.data(), Tensor::HALF);
            Tensor b = net.networkParameter(l, true, flat.data(), Tensor::HALF);
            std::cout << "layer " << l << " w " << w.size(0) << "x" << w.size(1) << " at "
                      << (static_cast<char*>(w.rawPtr()) - flat.data()) / 2 << " bias "
                      << (b.defined() ? (static_cast<char*>(b.rawPtr()) - flat.data()) / 2 : -1) << "\n";
        }
        Activation celu("celu");
        std::cout << "activation " << celu.id() << " code_bytes " << celu.code().size() << "\n";
        auto enc = EncodingFactory::Instance().create("{\"id\": \"Identity\", \"start_in\": 1, \"n_in\": 2}");
        std::cout << "factory " << enc->id() << " " << enc->numOutputChannels() << " " << enc->maxInputChannel() << "\n";
        std::cout << "forward_memory " << net.forwardMemory(100, 7) << " adjoint_memory " << net.adjointMemory(100, 7) << "\n";
        if (mode != "gpu") return 0;

        QuickMLP::Instance().checkCudaAvailable();
        const std::string dir = argv[3];
        const std::vector<float> x = readFloats(dir + "/x.bin"), adj = readFloats(dir + "/adj.bin"), p32 = readFloats(dir + "/params.bin");
        const int n = static_cast<int>(x.size()) / net.channelsIn();
        std::vector<__half> p16(p32.size());
        for (size_t i = 0; i < p32.size(); ++i) p16[i] = __float2half(p32[i]);
        Tensor params(Tensor::HALF, {net.networkParameterCount()}), grads(Tensor::FLOAT, {net.networkParameterCount()});
        Tensor input(Tensor::FLOAT, {n, net.channelsIn()}), output(Tensor::FLOAT, {n, net.channelsOut()});
        Tensor adjOutput(Tensor::FLOAT, {n, net.channelsOut()}), adjInput(Tensor::FLOAT, {n, net.channelsIn()});
        cudaMemcpy(params.rawPtr(), p16.data(), p16.size() * 2, cudaMemcpyHostToDevice);
        cudaMemcpy(input.rawPtr(), x.data(), x.size() * 4, cudaMemcpyHostToDevice);
        cudaMemcpy(adjOutput.rawPtr(), adj.data(), adj.size() * 4, cudaMemcpyHostToDevice);
        grads.zero_();
        adjInput.zero_();
        net.setNetworkParameter(params, Tensor::INFERENCE);
        net.setNetworkParameter(grads, Tensor::GRADIENTS);
        CUstream stream = nullptr;
        net.inference(input, output, stream);
        std::vector<float> out(static_cast<size_t>(n) * net.channelsOut());
        cudaMemcpy(out.data(), output.rawPtr(), out.size() * 4, cudaMemcpyDeviceToHost);
        writeRaw(dir + "/inference.bin", out);
        const int flags = FusedNetwork::GRADIENTS_INPUT | FusedNetwork::GRADIENTS_NETWORK_WEIGHTS;
        TmpMemory fwd(net.forwardMemory(input, flags)), bwd(net.adjointMemory(input, flags));
        output.zero_();
        net.forward(input, output, fwd.get(), stream);
        net.adjoint(input, adjOutput, flags, adjInput, fwd.get(), bwd.get(), stream);
        cudaDeviceSynchronize();
        cudaMemcpy(out.data(), output.rawPtr(), out.size() * 4, cudaMemcpyDeviceToHost);
        writeRaw(dir + "/forward.bin", out);
        std::vector<float> gi(x.size()), gw(p32.size());
        cudaMemcpy(gi.data(), adjInput.rawPtr(), gi.size() * 4, cudaMemcpyDeviceToHost);
        cudaMemcpy(gw.data(), grads.rawPtr(), gw.size() * 4, cudaMemcpyDeviceToHost);
        writeRaw(dir + "/adj_input.bin", gi);
        writeRaw(dir + "/grad_params.bin", gw);
        // a weight view of the bound gradient tensor shares its memory
        Tensor w0 = net.networkParameter(0, false, Tensor::GRADIENTS);
        std::cout << "grad_view " << (w0.rawPtr() == grads.rawPtr() ? "shared" : "copy") << "\n";
        net.zeroGradients();
        cudaMemcpy(gw.data(), grads.rawPtr(), gw.size() * 4, cudaMemcpyDeviceToHost);
        double s = 0;
        for (float v : gw) s += v < 0 ? -v : v;
        std::cout << "zeroed " << s << "\n";
        std::cout << "gpu ok\n";
        return 0;
    } catch (const std::exception& e) {
        std::cout << "exception " << e.what() << "\n";
        return 1;
    }
}
