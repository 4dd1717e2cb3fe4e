// The mounter's host side (llmoop_b200/csrc/package.cpp: manifest, tensor index, integrity table, kernel plan, tensor
// reads) as a stand-alone program, so that it can run under ASan / UBSan without a GPU.
// Usage: package_mount_cases <package directory>...   Prints "ok <dir> tensors=<n> ops=<n> bytes=<n>" per package that
// opens with full verification and whose every tensor reads back with a matching hash, or "error <dir>: <message>"
// (the mounter's own error text) and exits with the number of packages that failed.
#include <cstdio>
#include <exception>
#include <string>

#include "../llmoop_b200/csrc/package.hpp"

int main(int argc, char **argv) {
    int failures = 0;
    for (int i = 1; i < argc; i++) {
        try {
            const std::shared_ptr<nerve::HostPackage> package = nerve::HostPackage::open(argv[i], nerve::VerifyLevel::All);
            size_t bytes = 0, ops = 0;
            for (const auto &item : package->tensors()) bytes += package->read_tensor(item.first, true).size();
            const nerve::ModelPlan &plan = package->plan();
            for (const nerve::ComponentPlan &layer : plan.layers) ops += layer.ops.size();
            for (const nerve::ComponentPlan &layer : plan.draft_layers) ops += layer.ops.size();
            std::printf("ok %s tensors=%zu ops=%zu bytes=%zu\n", argv[i], package->tensors().size(), ops, bytes);
        } catch (const std::exception &error) {
            failures++;
            std::printf("error %s: %s\n", argv[i], error.what());
        }
    }
    return failures;
}
