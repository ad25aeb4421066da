// The loop that calls the optimizer: TrainingLoop.Run (autograd/training_loop.go:96-214).
// It groups micro-batches into updates, zeroes gradients at the start of a group, steps the
// optimizer and the schedule when a group is complete, reports at the logging cadence, and on
// cancellation drops unfinished gradients and hands the group's starting sampler position to Save.
#include <stdexcept>

#include "autograd.hpp"

namespace autograd {

std::string TrainingLoop::Run(bool* cancelled) {
    if (cancelled) *cancelled = false;
    if (!Next || Optimizer == nullptr || !Step) return "autograd: training loop needs a reader, an optimizer and a step";
    if (Updates < 0 || Applied < 0 || Applied > Updates) return "autograd: invalid training loop update count";
    const int groups = Accumulate < 2 ? 1 : Accumulate;
    if (groups > 1 && !Position) return "autograd: accumulation rewinds need a position sampler";
    GradAccumulator accumulator;
    std::string e = GradAccumulator::New(groups, &accumulator);
    if (!e.empty()) return e;
    const int every = LogEvery < 1 ? 25 : LogEvery;
    const int start = Applied;  // a resumed run reports its own first update, not the absolute first
    const bool captureStart = groups > 1 || (Position && Save);
    bool haveSavepoint = false, isStopped = false, stoppedByCancel = false, awaitingFirstBatch = false;
    std::string savepoint, stopped;
    try {
        while (Applied < Updates) {
            if (accumulator.Pending() == 0) {
                if (captureStart) {
                    savepoint.clear();
                    if (!(e = Position(&savepoint)).empty()) return e;
                    haveSavepoint = true;
                }
                Optimizer->ZeroGrad();
            }
            std::string err;
            int status = Next(&err);
            if (status == EndOfEpoch) {
                if (awaitingFirstBatch) {
                    status = Failed;
                    err = "autograd: training epoch contains no batches";
                } else {
                    if (NextEpoch && !(e = NextEpoch()).empty()) return e;
                    awaitingFirstBatch = true;
                    continue;
                }
            }
            if (status != Batch) {
                if (accumulator.Pending() != 0) {
                    // The partial gradients are dropped; the rewound position replays those
                    // micro-batches after a resume.
                    Optimizer->ZeroGrad();
                    accumulator.Reset();
                } else {
                    haveSavepoint = false;
                }
                stopped = err.empty() ? "autograd: the reader failed" : err;
                stoppedByCancel = status == Cancelled;
                isStopped = true;
                break;
            }
            awaitingFirstBatch = false;
            double loss = 0;
            err.clear();
            status = Step(accumulator.SeedScale(), &loss, &err);
            if (status != 0) {
                if (err.empty()) err = "autograd: the step failed";
                if (status != Cancelled) return err;
                Optimizer->ZeroGrad();
                accumulator.Reset();
                if (!haveSavepoint) {
                    if (cancelled) *cancelled = true;
                    return err;
                }
                stopped = err;
                stoppedByCancel = true;
                isStopped = true;
                break;
            }
            bool complete = false;
            if (!(e = accumulator.MicroBatch(nullptr, &complete)).empty()) return e;
            if (!complete) continue;
            haveSavepoint = false;  // a completed group leaves nothing to rewind
            Applied++;
            Optimizer->Step();
            if (Schedule != nullptr) Schedule->Step(*Optimizer);
            if ((Applied == start + 1 || Applied % every == 0 || Applied == Updates) && Report) Report(Applied, loss);
        }
    } catch (const std::exception& ex) {
        return ex.what();  // the reference's optimizer panics on a launch error; here it ends the run
    }
    if (!isStopped) return Save ? Save(nullptr) : "";
    if (!stoppedByCancel) return stopped;
    if (cancelled) *cancelled = true;
    if (Save) {
        e = Save(haveSavepoint ? &savepoint : nullptr);
        if (!e.empty()) return stopped + "\n" + e;
    }
    return stopped;
}

}  // namespace autograd
