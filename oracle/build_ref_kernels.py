"""GPU-side oracle: the reference's own fused kernels (inference, backward, weight update), built from the reference
checkout.  TEST INFRASTRUCTURE.

The reference ships its fused network as CUDA *templates with holes* (src_cpp/include/qmlp/kernels/network_forward.cuh)
that its host code fills per network and hands to NVRTC (FusedNetwork::compileInferenceKernel,
src_cpp/src/fused_network.cpp:392-505). The host library cannot be built here (its kernel-loader, json, magic_enum and
spdlog submodules are absent), but the kernel templates compile on their own. This script does, for one network
configuration, what compileInferenceKernel does: it reads the template where it lies in the reference checkout, fills
the holes by the rules of fused_network.cpp:353-462, appends a small launcher (ours) that reproduces the reference's
launch configuration (fused_network.cpp:472-485, 534-550) and constant upload (encoding_hashgrid.cpp:204-243), and
compiles the result for sm_100a into oracle/_ref/ (git-ignored: generated reference text and binaries never enter the
repository). Nothing here is imported by the product; only tests/ and bench.py's reference leg load what it builds.

The reference checkout is only needed when this script runs; the built libraries travel with the tree.
"""
import hashlib
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
OUT_DIR = os.path.join(ROOT, "oracle", "_ref")


def reference_dir():
    d = os.environ.get("QMLP_REFERENCE_DIR", os.path.normpath(os.path.join(ROOT, os.pardir, "reference")))
    return d if os.path.isdir(os.path.join(d, "src_cpp", "include", "qmlp", "kernels")) else None


def _round16(v):
    return (v + 15) // 16 * 16


def _activation_table(ref, cfg):
    with open(os.path.join(ref, "src_cpp", "include", "qmlp", "builtin-activations.json")) as f:
        table = {a["id"]: a for a in json.load(f)}
    for a in cfg.get("activations", []):          # user-defined snippets of the configuration
        if isinstance(a, dict):
            table[a["id"]] = a
    return table


def _activation_struct(a):
    # the form Activation::generateCode emits (src_cpp/src/activation.cpp:13-40)
    return ("struct %s {\n"
            "    static __device__ half forward(half x) { half z; %s ; return z; }\n"
            "    static __device__ half adjoint(half x, half adjz) { half adjx; %s ; return adjx; }\n"
            "};\n") % (a["id"], a["forward"], a["adjoint"])


def library_name(cfg, kind="inference"):
    return "libref_%s_%s.so" % (kind, hashlib.sha1(json.dumps(cfg, sort_keys=True).encode()).hexdigest()[:16])


def generate(cfg, ref, kind="inference"):
    """Fills network_forward.cuh (kind "inference") or network_backward.cuh (kind "backward") for `cfg` and appends the
    launcher. Returns CUDA source text."""
    kdir = os.path.join(ref, "src_cpp", "include", "qmlp", "kernels")
    template = {"inference": "network_forward.cuh", "backward": "network_backward.cuh",
                "wgrad": "network_weight_update_block.cuh"}[kind]
    with open(os.path.join(kdir, template)) as f:
        code = f.read()
    encs = cfg["encodings"]
    layers = cfg["network"]
    acts = _activation_table(ref, cfg)

    includes, constants, calls, adj_calls, uploads = [], [], [], [], []
    enc_channels, grid_slot = 0, 0
    for i, e in enumerate(encs):
        out = "encodingOutput%d" % enc_channels
        calls.append("auto %s = encodingOutput + %d;" % (out, enc_channels))
        if e["id"].lower() == "identity":
            includes.append('#include <qmlp/kernels/encoding_identity.cuh>')
            calls.append("qmlp::kernel::EncodingIdentity<%d, %d>::forward(encodingInput, %s);"
                         % (e["start_in"], e["n_in"], out))
            adj_calls.append("qmlp::kernel::EncodingIdentity<%d, %d>::template adjoint<true, true>(encodingInput, "
                             "adjEncodingOutput + %d, adjEncodingInput);" % (e["start_in"], e["n_in"], enc_channels))
            enc_channels += e["n_in"]
        elif e["id"].lower() == "hashgrid":
            includes.append('#include <qmlp/kernels/encoding_hashgrid.cuh>')
            d, l, f_ = e["n_in"], e["n_levels"], e["n_features_per_level"]
            mode = "ADD" if str(e.get("combination_mode", "concat")).lower() == "add" else "CONCAT"
            ctype = "qmlp::kernel::HashGridConfig<%d,%d>" % (d, l)
            cname = "cEncoding%d" % i
            constants.append("__constant__ %s %s;" % (ctype, cname))
            calls.append("qmlp::kernel::EncodingHashGrid<%d,%d,%d,%d,qmlp::kernel::LayerCombinationMode::%s>"
                         "::forward(encodingInput, %s, %s);" % (e["start_in"], d, l, f_, mode, out, cname))
            adj_calls.append("qmlp::kernel::EncodingHashGrid<%d,%d,%d,%d,qmlp::kernel::LayerCombinationMode::%s>"
                             "::template adjoint<true, true>(encodingInput, adjEncodingOutput + %d, adjEncodingInput, %s);"
                             % (e["start_in"], d, l, f_, mode, enc_channels, cname))
            uploads.append((grid_slot, ctype, cname, d, l))
            grid_slot += 1
            enc_channels += l * f_ if mode == "CONCAT" else f_
        else:
            raise ValueError("encoding not on the path: %s" % e["id"])

    # padded layer geometry and parameter offsets (src_cpp/src/fused_network.cpp:95-206): all weights, then all biases.
    # Layer 0 takes the encoded channels; the reference's host code derives that width from num_inputs (:95,102), which
    # is only right for identity encodings and would make its own hash-grid device code unusable in a fused network.
    cin = _round16(enc_channels)
    geo, off = [], 0
    for lc in layers:
        cout = _round16(lc["n_out"])
        geo.append(dict(cin=cin, cout=cout, bias=bool(lc.get("bias", False)), act=lc["activation"], w=off))
        off += cin * cout
        cin = cout
    for g in geo:
        if g["bias"]:
            g["b"] = off
            off += g["cout"]
    num_parameters = off
    max_channels = max(max(g["cin"], g["cout"]) for g in geo)

    layer_calls = []
    for g in geo:
        layer_calls.append(
            "qmlp::kernel::Layer<%d, %d, %d, %s, activations::%s>::template inference<false>(networkParameters+%d, %s, "
            "intermediateResultsWarp, nullptr);" % (g["cin"] // 16, g["cout"] // 16, max_channels, "true" if g["bias"] else "false",
                                                   g["act"], g["w"], ("networkParameters+%d" % g["b"]) if g["bias"] else "nullptr"))
    # backward: layers in reverse order, adjoint<true> also writes the delta of every layer (what the weight update
    # reads), stash offsets in halfs per point = sum of the previous layers' widths (fused_network.cpp:207-218, 783-806)
    adj_layer_calls, stash_off = [], 0
    for g in geo:
        g["stash"] = stash_off
        stash_off += g["cout"]
    for g in reversed(geo):
        adj_layer_calls.append(
            "qmlp::kernel::Layer<%d, %d, %d, %s, activations::%s>::template adjoint<true>(networkParameters+%d, %s, "
            "adjIntermediateResultsWarp, forwardTmpMemory + (%d*numel32 + 32*%d*globalWarpID), "
            "adjointTmpMemory + (%d*numel32 + 32*%d*globalWarpID));"
            % (g["cin"] // 16, g["cout"] // 16, max_channels, "true" if g["bias"] else "false", g["act"], g["w"],
               ("networkParameters+%d" % g["b"]) if g["bias"] else "nullptr", g["stash"], g["cout"], g["stash"], g["cout"]))
    used = []
    for g in geo:
        if g["act"] not in used:
            used.append(g["act"])

    code = code.replace("$$INCLUDES$$", "\n".join(dict.fromkeys(includes)))
    code = code.replace("$$ENCODING_CONSTANTS$$", "\n".join(constants))
    code = code.replace("$$DEFINE_ACTIVATIONS$$", "\n".join(_activation_struct(acts[a]) for a in used))
    code = code.replace("$$MAX_CHANNELS$", str(max_channels))      # the template spells this hole with one trailing '$'
    code = code.replace("$$INPUT_PAD_START$$", str(enc_channels))
    code = code.replace("$$CHANNELS_IN$$", str(geo[0]["cin"]))
    code = code.replace("$$CHANNELS_OUT$$", str(geo[-1]["cout"]))
    code = code.replace("$$HAS_INPUT_GRADIENTS$$", "true")
    code = code.replace("$$CALL_ENCODINGS$$", "\n".join(adj_calls if kind == "backward" else calls))
    code = code.replace("$$CALL_NETWORK_LAYERS$$", "\n".join(layer_calls if kind == "inference" else adj_layer_calls))
    import re
    left = re.findall(r"\$\$[A-Z_]+\$", code)
    if left:
        raise RuntimeError("unfilled holes left in the reference template: %s" % left)

    upload_code = []
    for slot, ctype, cname, d, l in uploads:
        upload_code.append("""
    {
        %(ctype)s h;
        std::memset(&h, 0, sizeof h);
        h.parametersForward = const_cast<float*>(grids[%(slot)d].table);
        h.parametersBackward = grids[%(slot)d].grad;
        for (int i = 0; i < %(l)d; ++i) {
            h.layers[i].memoryOffset = grids[%(slot)d].levels[4 * i + 0];
            h.layers[i].resolution = grids[%(slot)d].levels[4 * i + 1];
            h.layers[i].hashGridSize = grids[%(slot)d].levels[4 * i + 2];
            h.layers[i].hashed = grids[%(slot)d].levels[4 * i + 3] != 0;
        }
        for (int i = 0; i < %(d)d; ++i) {
            h.boundingBoxMin[i] = grids[%(slot)d].boxMin[i];
            h.boundingBoxInvSize[i] = grids[%(slot)d].boxInvSize[i];
        }
        e = cudaMemcpyToSymbol(%(cname)s, &h, sizeof h);
        if (e != cudaSuccess) return static_cast<int>(e);
    }""" % dict(ctype=ctype, slot=slot, l=l, d=d, cname=cname))

    launcher = """
// ---- launcher (not reference code): launch configuration of FusedNetwork::compileInferenceKernel / inference ----------
#include <cstring>
struct RefGrid { const float* table; float* grad; const int* levels; const float* boxMin; const float* boxInvSize; };

extern "C" int ref_num_parameters() { return %(np)d; }
extern "C" int ref_channels(int which) { return which == 0 ? %(nin)d : %(nout)d; }

// One inference of the reference kernel on device buffers (contiguous row-major fp32 input/output, fp16 parameters).
// `grids`: host array, one entry per hash-grid encoding in order (device pointer to the fp32 table; host arrays with the
// level table as 4 ints per level [memoryOffset, resolution, hashGridSize, hashed] and the bounding box).
// iterations > 0: the launch is repeated and *ms receives the mean device time of one launch (CUDA events).
extern "C" int ref_inference(int numel, const float* input, float* output, const void* parameters, const RefGrid* grids,
                             int iterations, float* ms, int* launchInfo)
{
    using namespace qmlp::kernel;
    cudaError_t e = cudaSuccess;
    %(uploads)s
    int minGrid = 0, best = 0;
    e = cudaOccupancyMaxPotentialBlockSize(&minGrid, &best, NetworkKernelInferenceAndForward, 0, 0);
    if (e != cudaSuccess) return static_cast<int>(e);
    cudaDeviceProp props;
    e = cudaGetDeviceProperties(&props, 0);
    if (e != cudaSuccess) return static_cast<int>(e);
    const int maxChannels = %(maxc)d;
    int block = best;
    int smem = block * maxChannels * 2;
    if (smem > static_cast<int>(props.sharedMemPerBlock)) {
        block = static_cast<int>(props.sharedMemPerBlock) / (maxChannels * 2);
        block = (block / 32) * 32;
        smem = block * maxChannels * 2;
    }
    int grid = (numel + block - 1) / block;
    if (grid > minGrid) grid = minGrid;
    if (grid < 1) grid = 1;
    if (launchInfo) { launchInfo[0] = grid; launchInfo[1] = block; launchInfo[2] = smem; }
    const int sizesIn[2] = {numel, %(nin)d}, stridesIn[2] = {%(nin)d, 1};
    const int sizesOut[2] = {numel, %(nout)d}, stridesOut[2] = {%(nout)d, 1};
    Tensor2Read<float> in(const_cast<float*>(input), sizesIn, stridesIn);
    Tensor2RW<float> out(output, sizesOut, stridesOut);
    const half* p = static_cast<const half*>(parameters);
    cudaEvent_t t0, t1;
    cudaEventCreate(&t0);
    cudaEventCreate(&t1);
    const int runs = iterations > 0 ? iterations : 1;
    cudaEventRecord(t0, 0);
    for (int i = 0; i < runs; ++i)
        NetworkKernelInferenceAndForward<<<grid, block, smem, 0>>>(numel, in, out, p, nullptr);
    cudaEventRecord(t1, 0);
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaEventSynchronize(t1);
    float total = 0.f;
    if (e == cudaSuccess) cudaEventElapsedTime(&total, t0, t1);
    if (ms) *ms = total / runs;
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    return static_cast<int>(e);
}
""" % dict(np=num_parameters, nin=cfg["num_inputs"], nout=layers[-1]["n_out"],
           uploads="".join(upload_code), maxc=max_channels)
    backward_launcher = """
// ---- launcher (not reference code): launch configuration of FusedNetwork::compileBackwardKernel / adjoint ------------
#include <cstring>
struct RefGrid { const float* table; float* grad; const int* levels; const float* boxMin; const float* boxInvSize; };

extern "C" int ref_num_parameters() { return %(np)d; }
extern "C" int ref_stash_halfs_per_point() { return %(stash)d; }

// Backward kernel of the reference with all three gradient kinds enabled: adjInput (N x Cin, fp32, accumulated),
// delta of every layer into adjTmp ((N32 x Cout_l) halfs per layer, layers in order), grid gradients accumulated into
// grids[i].grad. fwdTmp: pre-activations of every layer, (N32 x Cout_l) halfs per layer, layers in order.
// adjOutput must be (N x %(noutp)d), i.e. zero-padded to the padded output width: the kernel reads that many columns
// of every row whatever the tensor's width (network_backward.cuh:66-72).
extern "C" int ref_backward(int numel, const float* input, const float* adjOutput, float* adjInput, const void* parameters,
                            const void* fwdTmp, void* adjTmp, const RefGrid* grids, int* launchInfo, float* ms)
{
    using namespace qmlp::kernel;
    cudaError_t e = cudaSuccess;
    %(uploads)s
    int minGrid = 0, best = 0;
    e = cudaOccupancyMaxPotentialBlockSize(&minGrid, &best, NetworkKernelBackward, 0, 0);
    if (e != cudaSuccess) return static_cast<int>(e);
    cudaDeviceProp props;
    e = cudaGetDeviceProperties(&props, 0);
    if (e != cudaSuccess) return static_cast<int>(e);
    const int maxChannels = %(maxc)d;
    int block = best;
    int smem = block * maxChannels * 2;
    if (smem > static_cast<int>(props.sharedMemPerBlock)) {
        block = static_cast<int>(props.sharedMemPerBlock) / (maxChannels * 2);
        block = (block / 32) * 32;
        smem = block * maxChannels * 2;
    }
    int grid = (numel + block - 1) / block;
    if (grid > minGrid) grid = minGrid;
    if (grid < 1) grid = 1;
    if (launchInfo) { launchInfo[0] = grid; launchInfo[1] = block; launchInfo[2] = smem; }
    const int sizesIn[2] = {numel, %(nin)d}, stridesIn[2] = {%(nin)d, 1};
    const int sizesOut[2] = {numel, %(noutp)d}, stridesOut[2] = {%(noutp)d, 1};
    Tensor2Read<float> in(const_cast<float*>(input), sizesIn, stridesIn);
    Tensor2Read<float> adjOut(const_cast<float*>(adjOutput), sizesOut, stridesOut);
    Tensor2RW<float> adjIn(adjInput, sizesIn, stridesIn);
    cudaEvent_t t0, t1;
    cudaEventCreate(&t0);
    cudaEventCreate(&t1);
    cudaEventRecord(t0, 0);
    NetworkKernelBackward<<<grid, block, smem, 0>>>(numel, in, adjOut, adjIn, static_cast<const half*>(parameters),
                                                    static_cast<const half*>(fwdTmp), static_cast<half*>(adjTmp));
    cudaEventRecord(t1, 0);
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    float total = 0.f;
    if (e == cudaSuccess) cudaEventElapsedTime(&total, t0, t1);
    if (ms) *ms = total;
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    return static_cast<int>(e);
}
""" % dict(np=num_parameters, nin=cfg["num_inputs"], noutp=geo[-1]["cout"], uploads="".join(upload_code),
           maxc=max_channels, stash=stash_off)
    # weight update: one launch of WeightUpdateSingleBlockKernel per layer, a single thread block each
    # (src_cpp/src/fused_network.cpp:876-995 for the kernel names and shared memory, :1081-1144 for the launches)
    wgrad_calls = []
    for li, g in enumerate(geo):
        if li == 0:
            kname = ("WeightUpdateSingleBlockKernel<float, OHatTmpLoader<%d>, InputLoader<%d> >"
                     % (g["cout"] // 16, g["cin"] // 16))
            b_arg = "in"
        else:
            kname = ("WeightUpdateSingleBlockKernel<float, OHatTmpLoader<%d>, HiddenLoader<%d, activations::%s> >"
                     % (g["cout"] // 16, g["cin"] // 16, geo[li - 1]["act"]))
            b_arg = "const_cast<half*>(static_cast<const half*>(fwdTmp)) + static_cast<ptrdiff_t>(%d) * numel32" % geo[li - 1]["stash"]
        wgrad_calls.append("""
    {
        auto kernel = %(kname)s;
        const int perWarpIn = 2 * 32 * (%(cin)d + %(cout)d), perWarpOut = 4 * %(cin)d * %(cout)d;
        const int perWarp = perWarpIn > perWarpOut ? perWarpIn : perWarpOut;
        int minGrid = 0, best = 0;
        e = cudaOccupancyMaxPotentialBlockSize(&minGrid, &best, kernel, 0, 0);
        if (e != cudaSuccess) return static_cast<int>(e);
        int block = best, smem = best / 32 * perWarp;
        if (smem > static_cast<int>(props.sharedMemPerBlock)) {
            const int warps = static_cast<int>(props.sharedMemPerBlock) / perWarp;
            if (warps == 0) return -1;   // "Layer too large for block-wise weight update"
            block = warps * 32;
            smem = warps * perWarp;
        }
        if (launchInfo) { launchInfo[2 * %(li)d] = block; launchInfo[2 * %(li)d + 1] = smem; }
        kernel<<<1, block, smem, 0>>>(numel, gradWeights + %(w)d,
                                      static_cast<half*>(adjTmp) + static_cast<ptrdiff_t>(%(stash)d) * numel32, %(b_arg)s);
        e = cudaGetLastError();
        if (e != cudaSuccess) return static_cast<int>(e);
    }""" % dict(kname=kname, cin=g["cin"], cout=g["cout"], li=li, w=g["w"], stash=g["stash"], b_arg=b_arg))
    wgrad_launcher = """
// ---- launcher (not reference code): the weight-update launches of FusedNetwork::adjoint ------------------------------
#include <cstring>
struct RefGrid { const float* table; float* grad; const int* levels; const float* boxMin; const float* boxInvSize; };

extern "C" int ref_num_parameters() { return %(np)d; }
extern "C" int ref_num_layers() { return %(nl)d; }

// Weight gradients of every layer, accumulated into gradWeights (fp32, the flat parameter layout; biases untouched: the
// reference has no bias gradient). adjTmp: delta of every layer, fwdTmp: pre-activations of every layer, both
// (N32 x Cout_l) halfs per layer in layer order. launchInfo receives (block, shared memory) per layer.
extern "C" int ref_weight_update(int numel, const float* input, float* gradWeights, const void* fwdTmp, void* adjTmp,
                                 const RefGrid* grids, int* launchInfo, float* ms)
{
    using namespace qmlp::kernel;
    cudaError_t e = cudaSuccess;
    %(uploads)s
    cudaDeviceProp props;
    e = cudaGetDeviceProperties(&props, 0);
    if (e != cudaSuccess) return static_cast<int>(e);
    const ptrdiff_t numel32 = (numel + 31) / 32 * 32;
    const int sizesIn[2] = {numel, %(nin)d}, stridesIn[2] = {%(nin)d, 1};
    Tensor2Read<float> in(const_cast<float*>(input), sizesIn, stridesIn);
    cudaEvent_t t0, t1;
    cudaEventCreate(&t0);
    cudaEventCreate(&t1);
    cudaEventRecord(t0, 0);
    %(calls)s
    cudaEventRecord(t1, 0);
    e = cudaDeviceSynchronize();
    float total = 0.f;
    if (e == cudaSuccess) cudaEventElapsedTime(&total, t0, t1);
    if (ms) *ms = total;
    cudaEventDestroy(t0);
    cudaEventDestroy(t1);
    return static_cast<int>(e);
}
""" % dict(np=num_parameters, nl=len(geo), nin=cfg["num_inputs"], uploads="".join(upload_code), calls="".join(wgrad_calls))
    # tensor.cuh uses std::begin / std::copy and relies on its includer for <iterator>
    tail = {"inference": launcher, "backward": backward_launcher, "wgrad": wgrad_launcher}[kind]
    return "#include <iterator>\n#include <algorithm>\n#include <cstdint>\n#include <cstddef>\n" + code + tail


def build(cfg, force=False, kind="inference"):
    """Builds the reference inference (or backward) kernel for `cfg` into oracle/_ref/. Returns the library path, or
    None when the reference checkout is not on this machine and no earlier build is there."""
    path = os.path.join(OUT_DIR, library_name(cfg, kind))
    ref = reference_dir()
    if ref is None:
        return path if os.path.exists(path) else None
    os.makedirs(OUT_DIR, exist_ok=True)
    src = path[:-3] + ".cu"
    text = generate(cfg, ref, kind)
    if os.path.exists(path) and os.path.exists(src) and not force:
        with open(src) as f:
            if f.read() == text:      # built from exactly this source
                return path
    with open(src, "w") as f:
        f.write(text)
    nvcc = os.environ.get("QMLP_NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC",
           "-I", os.path.join(ref, "src_cpp", "include"), "-o", path, src]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building the reference kernel failed:\n" + r.stdout[-3000:] + r.stderr[-3000:])
    return path


def default_configs():
    """The configurations the GPU parity tests and the benchmark compare against the reference kernel."""
    sys.path.insert(0, os.path.join(ROOT, "quick-mlp_b200"))
    from qmlp import configs as specs
    return {"config1": specs.config1(), "config2": specs.config2(),
            "config3_small": specs.config3(log2_hashmap_size=14), "config3": specs.config3(),
            "config4": specs.config4(), "config5_small": specs.config5(log2_hashmap_size=12), "config5": specs.config5()}


BACKWARD_CONFIGS = ("config1", "config2", "config3_small", "config3", "config4")


def build_all():
    built = {}
    for name, cfg in default_configs().items():
        built[name] = build(cfg)
        if name in BACKWARD_CONFIGS:
            built[name + " (backward)"] = build(cfg, kind="backward")
            built[name + " (weight update)"] = build(cfg, kind="wgrad")
    return built


if __name__ == "__main__":
    for k, v in build_all().items():
        print(k, v)
