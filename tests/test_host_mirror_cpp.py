"""The C++ host mirror (ffai_b200/host/moe_layer.hpp) compiles, links against the library and turns the
reference's precondition traps (MoELayer.swift:109-118, :684) and the library's status codes into
exceptions.  No compute call is made: this runs without a GPU."""
import os
import subprocess
import textwrap

from ffai_b200 import capi

from conftest import ROOT

PROGRAM = textwrap.dedent(r"""
    #include <cstdio>
    #include <cstring>
    #include "moe_layer.hpp"
    using namespace ffai_host;

    template <typename F> static int status_of(F f, std::string* msg = nullptr) {
        try { f(); } catch (const Error& e) { if (msg) *msg = e.what(); return e.status; }
        return FFAI_OK;
    }

    int main() {
        int bad = 0;
        // MoERouter.init preconditions
        bad += status_of([] { MoERouter r(0, 1, MoEGatingMode::softmaxThenTopK); }) != FFAI_ERR_INVALID_ARG;
        bad += status_of([] { MoERouter r(4, 5, MoEGatingMode::topKThenSoftmax); }) != FFAI_ERR_INVALID_ARG;
        bad += status_of([] { MoERouter r(4, 2, MoEGatingMode::topKThenSoftmax, true, {0.f, 1.f}); }) != FFAI_ERR_INVALID_ARG;
        bad += status_of([] { MoERouter r(4, 2, MoEGatingMode::softmaxThenTopK, false, {0.f, 0.f, 0.f, 0.f}); }) != FFAI_OK;

        // a config the library rejects: the exception carries its status and its message
        ffai_moe_config cfg;
        std::memset(&cfg, 0, sizeof cfg);
        cfg.struct_size = 4;
        ffai_moe_weights w;
        std::memset(&w, 0, sizeof w);
        std::string msg;
        int rc = status_of([&] { MoELayer layer(cfg, w); }, &msg);
        bad += rc == FFAI_OK;
        bad += msg.find("ffai_moe_create") == std::string::npos;
        std::printf("create: %d %s\n", rc, msg.c_str());

        // a file that does not exist
        msg.clear();
        rc = status_of([&] { MoELayer layer = MoELayer::fromSafetensors("/nonexistent/model.safetensors", "model.layers.0.mlp",
                                                                         FFAI_ST_SWITCH_MLP, cfg); }, &msg);
        bad += rc == FFAI_OK;
        bad += msg.find("ffai_st_open") == std::string::npos;
        std::printf("open: %d %s\n", rc, msg.c_str());

        // operator wrappers: shape guards come back as exceptions, not as a launch
        MoERouter r(8, 2, MoEGatingMode::softmaxThenTopK);
        rc = status_of([&] { Ops::moeRouterTopK(nullptr, nullptr, nullptr, 1, r, nullptr); });
        bad += rc == FFAI_OK;
        rc = status_of([&] { Ops::gather(nullptr, nullptr, nullptr, 4, 64, nullptr); });
        bad += rc == FFAI_OK;

        // the aliases name the same type
        static_assert(std::is_same<GPTOSSMoELayer, MoELayer>::value && std::is_same<Qwen35MoEFFN, MoELayer>::value, "aliases");
        std::printf("bad=%d\n", bad);
        return bad;
    }
""")


def test_cpp_host_mirror_compiles_links_and_raises(ffai_lib, tmp_path):
    lib_path = capi.library_path() if hasattr(capi, "library_path") else os.path.join(ROOT, "ffai_b200", "lib", "libffai_cuda.so")
    lib_dir = os.path.dirname(str(lib_path))
    src = tmp_path / "mirror.cpp"
    src.write_text("#include <type_traits>\n" + PROGRAM)
    exe = tmp_path / "mirror"
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-I", str(ROOT / "include"), "-I", str(ROOT / "ffai_b200" / "host"),
                    "-o", str(exe), str(src), "-L", lib_dir, "-lffai_cuda", f"-Wl,-rpath,{lib_dir}"], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "bad=0" in out.stdout
