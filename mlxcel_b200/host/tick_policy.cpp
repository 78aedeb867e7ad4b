// Scheduler core: the per-tick decision as a pure function of a small state record, plus the
// token-budget split of a mixed (decode rows + one prefill chunk) step.
//
// Behavioural model: the reference's decide_tick (src/server/batch/tick_policy.rs:184-389):
//   * nothing active, nothing queued, nothing parked      -> Idle
//   * a speculative slice alternates with classic actions  (never two slices in a row while
//     classic work is waiting)
//   * with active rows: Preempt > Admit (batch not full, queue non-empty) > Decode
//   * a parked chunked prefill yields to decode until `prefill_grant_interval` decode ticks have
//     passed since its last grant; only one chunked prefill is parked at a time
// On B200 a decode step and a 512-token prefill chunk fit one forward pass, so when
// `mixed_steps` is set the Admit/Prefill grant is folded into the decode tick (MixedStep)
// instead of displacing it.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <string>

namespace py = pybind11;

namespace {

enum class TickAction : int {
  Idle = 0,
  Decode = 1,
  Prefill = 2,        // run (a piece of) a prefill alone
  MixedStep = 3,      // decode rows + one prefill chunk in one forward
  SpeculativeRound = 4,
  Preempt = 5,
};

struct TickState {
  int active_rows = 0;            // sequences in Decoding state
  int max_batch = 4;
  int queued = 0;                 // admitted-but-not-started requests in the queue
  bool parked_prefill = false;    // a chunked prefill is part-way through
  int decode_ticks_since_prefill_grant = 0;
  int prefill_grant_interval = 16;
  bool pending_preemption = false;
  bool speculative_ready = false; // a drafter-backed row can run a verify round
  bool last_was_speculative = false;
  bool mixed_steps = true;
  bool blocks_available = true;   // admission has KV room for the next queued request
};

struct TickDecision {
  TickAction action = TickAction::Idle;
  bool admit = false;        // start the next queued request in this tick
  bool grant_prefill = false;  // the parked prefill gets a chunk in this tick
};

TickDecision decide_tick(const TickState& s) {
  TickDecision d;
  const bool has_prefill_work = s.parked_prefill || (s.queued > 0 && s.blocks_available);
  if (s.active_rows == 0 && !has_prefill_work) {
    d.action = s.pending_preemption ? TickAction::Preempt : TickAction::Idle;
    return d;
  }
  if (s.active_rows == 0) {
    d.action = TickAction::Prefill;
    d.grant_prefill = s.parked_prefill;
    d.admit = !s.parked_prefill;
    return d;
  }
  // active rows exist
  if (s.pending_preemption) {
    d.action = TickAction::Preempt;
    return d;
  }
  const bool classic_waiting = has_prefill_work;
  if (s.speculative_ready && !(s.last_was_speculative && classic_waiting)) {
    d.action = TickAction::SpeculativeRound;
    return d;
  }
  const bool batch_has_room = s.active_rows + (s.parked_prefill ? 1 : 0) < s.max_batch;
  if (s.parked_prefill) {
    const bool due = s.decode_ticks_since_prefill_grant >= s.prefill_grant_interval;
    if (s.mixed_steps) {
      d.action = TickAction::MixedStep;
      d.grant_prefill = true;
    } else if (due) {
      d.action = TickAction::Prefill;
      d.grant_prefill = true;
    } else {
      d.action = TickAction::Decode;
    }
    return d;
  }
  if (s.queued > 0 && s.blocks_available && batch_has_room) {
    d.admit = true;
    d.action = s.mixed_steps ? TickAction::MixedStep : TickAction::Prefill;
    return d;
  }
  d.action = TickAction::Decode;
  return d;
}

// Split a per-step token budget: decode rows take one token each, the rest (at most
// `chunk`) goes to the prefill piece. Returns the prefill piece length.
int prefill_piece(int token_budget, int decode_rows, int chunk_alone, int chunk_contended,
                  int remaining_prompt) {
  const int chunk = decode_rows > 0 ? chunk_contended : chunk_alone;
  int room = token_budget - decode_rows;
  if (room < 0) room = 0;
  return std::max(0, std::min({chunk, room, remaining_prompt}));
}

}  // namespace

void bind_scheduler(py::module_& m) {
  py::enum_<TickAction>(m, "TickAction")
      .value("Idle", TickAction::Idle)
      .value("Decode", TickAction::Decode)
      .value("Prefill", TickAction::Prefill)
      .value("MixedStep", TickAction::MixedStep)
      .value("SpeculativeRound", TickAction::SpeculativeRound)
      .value("Preempt", TickAction::Preempt);
  py::class_<TickState>(m, "TickState")
      .def(py::init<>())
      .def_readwrite("active_rows", &TickState::active_rows)
      .def_readwrite("max_batch", &TickState::max_batch)
      .def_readwrite("queued", &TickState::queued)
      .def_readwrite("parked_prefill", &TickState::parked_prefill)
      .def_readwrite("decode_ticks_since_prefill_grant", &TickState::decode_ticks_since_prefill_grant)
      .def_readwrite("prefill_grant_interval", &TickState::prefill_grant_interval)
      .def_readwrite("pending_preemption", &TickState::pending_preemption)
      .def_readwrite("speculative_ready", &TickState::speculative_ready)
      .def_readwrite("last_was_speculative", &TickState::last_was_speculative)
      .def_readwrite("mixed_steps", &TickState::mixed_steps)
      .def_readwrite("blocks_available", &TickState::blocks_available);
  py::class_<TickDecision>(m, "TickDecision")
      .def_readonly("action", &TickDecision::action)
      .def_readonly("admit", &TickDecision::admit)
      .def_readonly("grant_prefill", &TickDecision::grant_prefill);
  m.def("decide_tick", &decide_tick);
  m.def("prefill_piece", &prefill_piece, py::arg("token_budget"), py::arg("decode_rows"),
        py::arg("chunk_alone") = 2048, py::arg("chunk_contended") = 512,
        py::arg("remaining_prompt") = 1 << 30);
}
