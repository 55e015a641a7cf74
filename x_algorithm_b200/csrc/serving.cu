// Host-side serving duties that sit between the wire layer and the engine seam: the bounded request queue with
// staleness / deadline drops (phoenix/crates/serving/xai-recsys-engine/src/request_queue.rs:10-155) and deadline-aware
// admission control (admission.rs:44-227).  Plain C++ behind the C ABI; no GPU work, no threads of its own: the host
// calls phx_queue_dequeue from its dispatch loop where the reference awaits `server.dequeue()`.
#include <stdint.h>

#include <algorithm>
#include <chrono>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

#include "../../include/phoenix_b200.h"

namespace {
struct Item { uint64_t id, enqueue_us, deadline_us; };   // deadline_us 0 = none

// request_queue.rs:18-27
bool is_expired(const Item& it, uint64_t max_staleness_us, uint64_t now_us) {
  if (it.deadline_us != 0) return now_us > it.deadline_us;
  if (max_staleness_us == UINT64_MAX) return false;
  const uint64_t age = now_us > it.enqueue_us ? now_us - it.enqueue_us : 0;   // saturating_duration_since
  return age > max_staleness_us;
}
uint64_t sat_add(uint64_t a, uint64_t b) { return a > UINT64_MAX - b ? UINT64_MAX : a + b; }
uint64_t sat_mul(uint64_t a, uint64_t b) { return (b != 0 && a > UINT64_MAX / b) ? UINT64_MAX : a * b; }
}  // namespace

struct phx_request_queue {
  std::mutex mu;
  std::deque<Item> channel;     // the bounded channel the producers send into
  std::vector<Item> buffer;     // the batch under construction (capacity batch_size)
  std::vector<uint64_t> dropped;
  size_t batch_size = 1, channel_size = 1;
  uint64_t max_staleness_us = UINT64_MAX, batch_wait_us = 0;
  uint64_t total_dropped = 0;
};

struct phx_admission {
  std::mutex mu;
  phx_admission_config cfg;
  uint64_t service_time_us = 0, pipeline_time_us = 0;
};

namespace {
// the background task of the reference (request_queue.rs:58-93): channel -> buffer, expired items dropped on the way
void pump(phx_request_queue* q, uint64_t now_us) {
  while (!q->channel.empty() && q->buffer.size() < q->batch_size) {
    const Item it = q->channel.front();
    q->channel.pop_front();
    if (is_expired(it, q->max_staleness_us, now_us)) { q->dropped.push_back(it.id); q->total_dropped++; continue; }
    q->buffer.push_back(it);
  }
}
uint64_t ewma(uint64_t prev, uint64_t sample, double alpha) {   // admission.rs:97-103
  return prev == 0 ? sample : (uint64_t)(alpha * (double)sample + (1.0 - alpha) * (double)prev);
}
uint64_t queue_wait_us(const phx_admission* a, uint64_t q) {   // admission.rs:146-153
  return a->service_time_us == 0 ? 0 : sat_mul(q, a->service_time_us) / a->cfg.batch_size;
}
bool predicted_eta(const phx_admission* a, int64_t queue_depth, int model, uint64_t* eta) {
  const uint64_t q = queue_depth > 0 ? (uint64_t)queue_depth : 0;
  if (model == 0) {   // loop model, admission.rs:181-194
    if (a->service_time_us == 0) return false;
    const uint64_t batches_ahead = (q + 1 + a->cfg.batch_size - 1) / a->cfg.batch_size;
    *eta = sat_add(sat_mul(sat_add(batches_ahead, a->cfg.pipeline_depth), a->service_time_us), a->cfg.post_us);
    return true;
  }
  if (a->pipeline_time_us == 0) return false;   // pipeline model, admission.rs:196-202
  *eta = sat_add(sat_add(queue_wait_us(a, q), a->pipeline_time_us), a->cfg.post_us);
  return true;
}
}  // namespace

extern "C" {

uint64_t phx_now_us(void) {
  return (uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

phx_status phx_queue_create(int32_t batch_size, int32_t channel_size, uint64_t max_staleness_us, uint64_t batch_wait_us,
                            phx_request_queue** out) {
  if (!out || batch_size <= 0 || channel_size <= 0) return PHX_E_ARG;
  phx_request_queue* q = new phx_request_queue();
  q->batch_size = (size_t)batch_size; q->channel_size = (size_t)channel_size;
  q->max_staleness_us = max_staleness_us; q->batch_wait_us = batch_wait_us;
  q->buffer.reserve(q->batch_size);
  *out = q;
  return PHX_OK;
}

void phx_queue_destroy(phx_request_queue* q) { delete q; }

phx_status phx_queue_push(phx_request_queue* q, uint64_t request_id, uint64_t enqueue_time_us, uint64_t deadline_us) {
  if (!q) return PHX_E_ARG;
  std::lock_guard<std::mutex> lk(q->mu);
  if (q->channel.size() >= q->channel_size) return PHX_E_CAPACITY;
  q->channel.push_back(Item{request_id, enqueue_time_us, deadline_us});
  return PHX_OK;
}

phx_status phx_queue_dequeue(phx_request_queue* q, uint64_t now_us, uint64_t* ids_out, int32_t max_out, int32_t* n_out,
                             uint64_t* dropped_out, int32_t max_dropped, int32_t* n_dropped) {
  if (!q || !ids_out || !n_out || max_out < (int32_t)q->batch_size) return PHX_E_ARG;
  std::vector<Item> items;
  items.reserve(q->batch_size);
  std::unique_lock<std::mutex> lk(q->mu);
  pump(q, now_us);
  items.swap(q->buffer);                       // request_queue.rs:111-118: the whole buffer at once
  q->buffer.reserve(q->batch_size);
  if (q->batch_wait_us > 0) {
    // wait_for_batch (request_queue.rs:139-155): poll every millisecond until the batch is full (or, from an empty
    // start, holds one request) or the wait is over; `now_us` advances with the real clock meanwhile
    const uint64_t t0 = phx_now_us(), end = t0 + q->batch_wait_us;
    const size_t target = items.empty() ? 1 : q->batch_size;
    while (items.size() < target) {
      const uint64_t t = phx_now_us();
      if (t >= end) break;
      lk.unlock();
      std::this_thread::sleep_for(std::chrono::microseconds(std::min<uint64_t>(end - t, 1000)));
      lk.lock();
      pump(q, now_us + (phx_now_us() - t0));
      const size_t k = std::min(q->batch_size - items.size(), q->buffer.size());
      items.insert(items.end(), q->buffer.begin(), q->buffer.begin() + k);
      q->buffer.erase(q->buffer.begin(), q->buffer.begin() + k);
    }
    now_us += phx_now_us() - t0;
  }
  int n = 0;
  for (const Item& it : items) {               // request_queue.rs:124-135: a last freshness check on the way out
    if (is_expired(it, q->max_staleness_us, now_us)) { q->dropped.push_back(it.id); q->total_dropped++; }
    else ids_out[n++] = it.id;
  }
  *n_out = n;
  int nd = 0;
  if (dropped_out && n_dropped) {
    for (; nd < max_dropped && nd < (int)q->dropped.size(); ++nd) dropped_out[nd] = q->dropped[nd];
    q->dropped.erase(q->dropped.begin(), q->dropped.begin() + nd);
    *n_dropped = nd;
  } else {
    q->dropped.clear();
    if (n_dropped) *n_dropped = 0;
  }
  return PHX_OK;
}

phx_status phx_queue_stats(phx_request_queue* q, int32_t* waiting, uint64_t* total_dropped) {
  if (!q) return PHX_E_ARG;
  std::lock_guard<std::mutex> lk(q->mu);
  if (waiting) *waiting = (int32_t)(q->channel.size() + q->buffer.size());
  if (total_dropped) *total_dropped = q->total_dropped;
  return PHX_OK;
}

phx_status phx_admission_create(const phx_admission_config* cfg, phx_admission** out) {
  if (!cfg || !out || (cfg->eta_model != 0 && cfg->eta_model != 1)) return PHX_E_ARG;
  phx_admission* a = new phx_admission();
  a->cfg = *cfg;
  if (!(a->cfg.ewma_alpha > 0.0 && a->cfg.ewma_alpha <= 1.0)) a->cfg.ewma_alpha = 0.2;   // admission.rs:74-78
  if (a->cfg.batch_size < 1) a->cfg.batch_size = 1;
  *out = a;
  return PHX_OK;
}

void phx_admission_destroy(phx_admission* a) { delete a; }

phx_status phx_admission_set_enabled(phx_admission* a, int32_t on) {
  if (!a) return PHX_E_ARG;
  std::lock_guard<std::mutex> lk(a->mu);
  a->cfg.enabled = on != 0;
  return PHX_OK;
}

phx_status phx_admission_reset(phx_admission* a) {
  if (!a) return PHX_E_ARG;
  std::lock_guard<std::mutex> lk(a->mu);
  a->service_time_us = a->pipeline_time_us = 0;
  return PHX_OK;
}

phx_status phx_admission_record_service_us(phx_admission* a, uint64_t sample_us) {
  if (!a) return PHX_E_ARG;
  if (sample_us == 0) return PHX_OK;
  std::lock_guard<std::mutex> lk(a->mu);
  a->service_time_us = ewma(a->service_time_us, sample_us, a->cfg.ewma_alpha);
  return PHX_OK;
}

phx_status phx_admission_record_sojourn_us(phx_admission* a, uint64_t sample_us, int64_t admit_backlog) {
  if (!a) return PHX_E_ARG;
  std::lock_guard<std::mutex> lk(a->mu);
  if (a->cfg.eta_model != 1 || sample_us == 0) return PHX_OK;   // admission.rs:130-133
  const uint64_t wait = queue_wait_us(a, admit_backlog > 0 ? (uint64_t)admit_backlog : 0);
  const uint64_t residual = sample_us > wait ? sample_us - wait : 0;
  if (residual == 0) return PHX_OK;
  a->pipeline_time_us = ewma(a->pipeline_time_us, residual, a->cfg.ewma_alpha);
  return PHX_OK;
}

int32_t phx_admission_predicted_eta_us(phx_admission* a, int64_t queue_depth, int32_t model, uint64_t* eta_us) {
  if (!a || !eta_us) return 0;
  std::lock_guard<std::mutex> lk(a->mu);
  return predicted_eta(a, queue_depth, model < 0 ? a->cfg.eta_model : model, eta_us) ? 1 : 0;
}

int32_t phx_admission_should_reject(phx_admission* a, int64_t remaining_us, int64_t queue_depth) {
  if (!a) return 0;
  std::lock_guard<std::mutex> lk(a->mu);
  if (!a->cfg.enabled) return 0;                                  // admission.rs:155-175
  const uint64_t q = queue_depth > 0 ? (uint64_t)queue_depth : 0;
  if (q < a->cfg.batch_size) return 0;
  if (remaining_us < 0) return 0;                                  // no deadline: admit
  uint64_t eta = 0;
  if (!predicted_eta(a, queue_depth, a->cfg.eta_model, &eta)) return 0;
  return sat_add(eta, a->cfg.margin_us) > (uint64_t)remaining_us ? 1 : 0;
}

phx_status phx_admission_estimates(phx_admission* a, uint64_t* service_time_us, uint64_t* pipeline_time_us) {
  if (!a) return PHX_E_ARG;
  std::lock_guard<std::mutex> lk(a->mu);
  if (service_time_us) *service_time_us = a->service_time_us;
  if (pipeline_time_us) *pipeline_time_us = a->pipeline_time_us;
  return PHX_OK;
}

}  // extern "C"
