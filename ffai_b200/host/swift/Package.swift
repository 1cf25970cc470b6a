// swift-tools-version:5.9
// SwiftPM package that puts libffai_cuda behind FFAI's MoE-layer call surface.
// Shipped as source: no Swift toolchain exists where the CUDA library is built and tested.
import PackageDescription

let package = Package(
    name: "FFAICuda",
    products: [.library(name: "FFAICuda", targets: ["FFAICuda"])],
    targets: [
        // C module over the shared library; its umbrella header includes include/ffai_cuda.h.
        .systemLibrary(name: "CFFAICuda", path: "Sources/CFFAICuda"),
        .target(name: "FFAICuda", dependencies: ["CFFAICuda"],
                linkerSettings: [.linkedLibrary("ffai_cuda")]),
    ]
)
