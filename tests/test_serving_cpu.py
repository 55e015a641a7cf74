"""Request queue and admission control (no GPU).  The admission cases are the reference's own unit tests
(xai-recsys-engine/src/admission.rs:229-414) re-typed against the C ABI; the queue cases follow the rules of
request_queue.rs:18-27, 58-135."""
import pytest

from x_algorithm_b200.serving import AdmissionController, RequestQueue, NEVER


def test_admission_known_answers_of_the_reference_tests():
    c = AdmissionController(enabled=False)
    c.record_service_time_us(100_000)
    assert not c.should_reject(1, 1_000_000)                       # disabled_never_rejects
    c = AdmissionController()
    assert not c.should_reject(1, 1_000_000)                       # no_estimate_admits
    c.record_service_time_us(100_000)
    assert not c.should_reject(None, 1_000_000)                    # missing_deadline_without_fallback_admits
    assert c.should_reject(500_000, 320)                           # deep_backlog_tight_deadline_rejects
    assert not c.should_reject(500_000, 0)                         # light_load_admits
    assert not c.should_reject(1, 10)                              # shallow_backlog_below_floor_admits
    c = AdmissionController(fallback_budget_us=300_000)            # fallback_budget_exposed_and_used
    assert c.fallback_budget_us == 300_000
    c.record_service_time_us(100_000)
    assert c.should_reject(300_000, 320)
    assert AdmissionController().fallback_budget_us is None        # fallback_budget_none_when_disabled
    c = AdmissionController(pipeline_depth=1)                      # pipeline_depth_adds_completion_lag
    c.record_service_time_us(100_000)
    assert c.predicted_eta_us(0) == 200_000 and c.predicted_eta_us(320) == 1_200_000
    bad = AdmissionController(pipeline_depth=1)
    bad.record_service_time_us(500_000)
    assert bad.predicted_eta_us(32) == 1_500_000 and bad.should_reject(1_200_000, 32)
    c = AdmissionController()                                      # predicted_eta_tracks_backlog
    assert c.predicted_eta_us(100) is None
    c.record_service_time_us(100_000)
    assert c.service_time_us() == 100_000
    assert c.predicted_eta_us(0) == 100_000 and c.predicted_eta_us(320) == 1_100_000 and c.predicted_eta_us(-5) == 100_000
    c = AdmissionController(eta_model="pipeline")                  # sojourn_replaces_pipeline_depth_term
    c.record_service_time_us(23_000)
    c.record_sojourn_us(80_000, 9)
    p = 80_000 - 9 * 23_000 // 32
    assert c.pipeline_time_us() == p
    assert c.predicted_eta_us(0) == p and c.predicted_eta_us(9) == 80_000 and c.predicted_eta_us(32) == 23_000 + p
    c = AdmissionController(eta_model="pipeline")                  # sojourn_deep_queue_stores_residual
    c.record_service_time_us(100_000)
    c.record_sojourn_us(500_000, 32)
    assert c.pipeline_time_us() == 400_000 and c.predicted_eta_us(0) == 400_000 and c.predicted_eta_us(32) == 500_000
    c = AdmissionController(eta_model="pipeline")                  # sojourn_without_s_is_just_p
    c.record_sojourn_us(75_000, 0)
    assert c.predicted_eta_us(40) == 75_000
    c = AdmissionController()                                      # loop_model_ignores_sojourn_samples
    c.record_service_time_us(100_000)
    c.record_sojourn_us(80_000, 0)
    assert c.pipeline_time_us() == 0 and c.predicted_eta_us(0) == 100_000
    assert c.predicted_eta_us(0, "loop") == 100_000 and c.predicted_eta_us(0, "pipeline") is None
    c = AdmissionController(eta_model="rust")                      # reset_estimates_clears_s_and_p; alias of "pipeline"
    c.record_service_time_us(100_000)
    c.record_sojourn_us(80_000, 0)
    assert c.service_time_us() > 0 and c.pipeline_time_us() > 0 and c.should_reject(1, 32)
    c.reset_estimates()
    assert c.service_time_us() == 0 and c.pipeline_time_us() == 0 and not c.should_reject(1, 32)
    with pytest.raises(ValueError):                                # eta_model_parses_aliases
        AdmissionController(eta_model="nope")
    AdmissionController(eta_model="python")
    c = AdmissionController()                                      # ewma_is_idle_independent_and_smooths
    c.record_service_time_us(100_000)
    c.record_service_time_us(800_000)
    assert c.service_time_us() == int(0.2 * 800_000 + 0.8 * 100_000)
    assert not c.should_reject(500_000, 32)
    c.set_enabled(False)
    assert not c.should_reject(1, 1 << 40)


def test_queue_batches_in_arrival_order_and_bounds_its_channel():
    q = RequestQueue(batch_size=4, channel_size=6)
    assert all(q.push(i, 1000 + i) for i in range(6))
    assert not q.push(99, 2000)                                    # channel full: the caller sheds
    ids, dropped = q.dequeue(now=5000)
    assert ids == [0, 1, 2, 3] and dropped == []
    assert q.waiting() == 2
    assert q.push(6, 5001)
    ids, dropped = q.dequeue(now=6000)
    assert ids == [4, 5, 6] and dropped == []
    assert q.dequeue(now=7000) == ([], [])


def test_queue_drops_expired_requests_and_reports_them():
    # without a deadline: older than max_staleness (strictly) -> dropped; the deadline, when given, decides alone
    q = RequestQueue(batch_size=8, channel_size=16, max_staleness_us=1000)
    q.push(1, 0)                     # age 1500 at dequeue: stale
    q.push(2, 600)                   # age 900: fresh
    q.push(3, 500)                   # age exactly 1000: not older than the bound, kept
    q.push(4, 0, deadline_us=2000)   # old, but its deadline is still ahead: kept
    q.push(5, 1400, deadline_us=1499)  # young, but past its deadline: dropped
    ids, dropped = q.dequeue(now=1500)
    assert ids == [2, 3, 4] and sorted(dropped) == [1, 5]
    # no staleness bound: nothing expires without a deadline
    q = RequestQueue(batch_size=2, channel_size=4, max_staleness_us=NEVER)
    q.push(7, 0)
    assert q.dequeue(now=10**15) == ([7], [])
    # a request can expire between being batched and being handed out: first call leaves it in the batch buffer
    q = RequestQueue(batch_size=2, channel_size=8, max_staleness_us=100)
    for i in range(3):
        q.push(10 + i, 0)
    ids, dropped = q.dequeue(now=50)
    assert ids == [10, 11] and dropped == []
    ids, dropped = q.dequeue(now=500)
    assert ids == [] and dropped == [12]


def test_queue_batch_wait_fills_up_from_late_arrivals():
    import threading
    import time
    q = RequestQueue(batch_size=3, channel_size=8, batch_wait_us=200_000)
    q.push(1, 0)

    def late():
        time.sleep(0.02)
        q.push(2, 0); q.push(3, 0)
    t = threading.Thread(target=late)
    t.start()
    t0 = time.perf_counter()
    ids, _ = q.dequeue(now=0)
    dt = time.perf_counter() - t0
    t.join()
    assert ids == [1, 2, 3] and dt < 0.15          # returned as soon as the batch was full, not after the whole wait
    t0 = time.perf_counter()
    assert q.dequeue(now=0) == ([], [])            # nothing arrives: gives up after the wait
    assert 0.15 < time.perf_counter() - t0 < 1.0
