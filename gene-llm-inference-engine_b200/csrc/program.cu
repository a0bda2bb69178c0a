// Launch programs: a recorded sequence of this library's launches, repeated with one call.
//
// A step of the model launches a hundred or more kernels; what the host does for each of them (checking
// tensors, converting arguments, choosing a plan) costs several times the launch itself, and a prompt
// portion of a few hundred tokens is over on the device before the host has issued it. The launch
// sequence of a part depends only on a few numbers of the step (its token count, how its rows split
// between the attention kernels), so the caller records it once per such shape and replays it. The
// reference's device model has this loop in C++ for the same reason (src/gpu/gpu_transformer.cpp:379-426).
#include "common.cuh"

namespace gi {
thread_local Program* tl_recording = nullptr;
}

using namespace gi;

extern "C" {

// Starts recording on the calling thread. Recordings do not nest.
int gi_program_begin() {
    GI_REQUIRE(tl_recording == nullptr, "program_begin: a program is already being recorded on this thread");
    tl_recording = new Program();
    return 0;
}

// Ends the recording and hands the program to the caller (nullptr when none was being recorded).
void* gi_program_end() {
    Program* p = tl_recording;
    tl_recording = nullptr;
    return p;
}

int gi_program_size(const void* program) { return program ? static_cast<int>(static_cast<const Program*>(program)->calls.size()) : 0; }

// Repeats every recorded launch, in order, on ``stream``. Stops at the first entry point that fails.
int gi_program_run(void* program, void* stream) {
    GI_REQUIRE(program != nullptr, "program_run: no program");
    GI_REQUIRE(tl_recording == nullptr, "program_run: a program is being recorded on this thread");
    for (auto& call : static_cast<Program*>(program)->calls) {
        const int rc = call(stream);
        if (rc != 0) return rc;
    }
    return 0;
}

int gi_program_free(void* program) {
    delete static_cast<Program*>(program);
    return 0;
}

}  // extern "C"
