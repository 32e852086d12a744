"""`MetricsLogger` (history, backends, per-process behaviour, OpenTelemetry gauges through a fake meter) and
`Profiler` (window arithmetic, one active profiler per process, rank gating) with the tracing calls stubbed."""
import json
import os

import numpy as np
import pytest
import torch

from tunix_b200.sft import metrics_logger as ml, profiler as prof


class Recording:
  def __init__(self, fail=False):
    self.events, self.closed, self.fail = [], 0, fail

  def log_scalar(self, event, value, **kw):
    if self.fail:
      raise OSError("disk full")
    self.events.append((event, float(value), kw.get("step")))

  def close(self):
    self.closed += 1


def test_history_means_and_the_geometric_mean_of_perplexity():
  lg = ml.MetricsLogger()
  for step, (loss, ppl) in enumerate([(2.0, 4.0), (1.0, 16.0)]):
    lg.log("actor", "loss", torch.tensor(loss), ml.Mode.TRAIN, step)
    lg.log("actor", "perplexity", np.float32(ppl), "train", step)
  lg.log("actor", "loss", [1.0, 3.0], ml.Mode.EVAL, 0)                       # non-scalars are averaged
  assert lg.get_metric("actor", "loss", "train") == 1.5 and lg.get_metric("actor", "loss", ml.Mode.EVAL) == 2.0
  assert lg.get_metric("actor", "perplexity", "train") == pytest.approx(8.0)  # sqrt(4 * 16)
  assert lg.get_metric_history("actor", "loss", "train").tolist() == [2.0, 1.0]
  assert lg.metric_exists("actor", "loss", "eval") and not lg.metric_exists("critic", "loss", "train")
  with pytest.raises(ValueError, match="not found"):
    lg.get_metric("actor", "nope", "train")
  with pytest.raises(ValueError, match=r"Available metrics for mode 'train': \['loss', 'perplexity'\]"):
    lg.get_metric_history("actor", "nope", "train")
  lg.close()


def test_custom_backends_replace_the_defaults_and_a_failing_one_is_isolated(tmp_path, caplog):
  good, bad = Recording(), Recording(fail=True)
  opts = ml.MetricsLoggerOptions(log_dir=str(tmp_path), backend_kwargs={"custom_backend": [lambda: bad, lambda: good]})
  lg = ml.MetricsLogger(opts)
  with caplog.at_level("ERROR"):
    lg.log("", "loss", 0.5, "train", 7)
  assert good.events == [("/train/loss", 0.5, 7)] and "Recording" in caplog.text
  assert lg.get_metric("", "loss", "train") == 0.5                           # the history does not depend on backends
  assert not os.listdir(tmp_path)                                            # no default backend was created
  lg.close(); lg.close()
  assert good.closed == 1 and bad.closed == 1


def test_default_backends_write_jsonl_and_only_on_the_first_process(tmp_path, monkeypatch):
  opts = ml.MetricsLoggerOptions(log_dir=str(tmp_path / "a"), flush_every_n_steps=1)
  lg = ml.MetricsLogger(opts)
  lg.log("actor", "loss", 1.25, "train", 3)
  lg.close()
  lines = [json.loads(l) for l in open(tmp_path / "a" / "metrics.jsonl")]
  assert lines[0]["event"] == "actor/train/loss" and lines[0]["value"] == 1.25 and lines[0]["step"] == 3
  monkeypatch.setattr(ml, "_process_index", lambda: 1)
  other = ml.MetricsLogger(ml.MetricsLoggerOptions(log_dir=str(tmp_path / "b")))
  other.log("actor", "loss", 1.0, "train", 0)
  assert not (tmp_path / "b").exists() and other.get_metric("actor", "loss", "train") == 1.0
  # options are plain data: two loggers from one options object do not share backends
  monkeypatch.setattr(ml, "_process_index", lambda: 0)
  first, second = ml.MetricsLogger(opts), ml.MetricsLogger(opts)
  assert first._backends[0] is not second._backends[0]
  first.close(); second.close()


class FakeMeter:
  def __init__(self):
    self.gauges = {}

  def get_meter(self, name):
    return self

  def create_gauge(self, name, unit="", description=""):
    self.gauges[name] = []
    outer = self

    class Gauge:
      def set(self, value, attributes=None):
        outer.gauges[name].append((value, dict(attributes or {})))
    return Gauge()


def test_opentelemetry_gauges_get_normalised_names_and_a_step_gauge(tmp_path):
  meter = FakeMeter()
  opts = ml.MetricsLoggerOptions(log_dir=str(tmp_path), enable_opentelemetry=True,
                                 backend_kwargs={"custom_backend": [Recording]})
  lg = ml.MetricsLogger(opts, otel_meter_provider=meter)
  lg.log("actor", "loss", 2.0, "train", 5)
  lg.log("actor", "rewards/mean score!", 0.5, "eval", 5)
  assert meter.gauges["tunix.training.loss"] == [(2.0, {"tunix.metrics_prefix": "actor", "tunix.mode": "train"})]
  assert "tunix.rewards.mean.score" in meter.gauges
  assert [v for v, _ in meter.gauges["tunix.training.step"]] == [5, 5]
  assert ml._otel_name("grad_norm") == "tunix.training.gradient.norm" and ml._otel_name("///") == "tunix.unnamed"
  quiet = ml.MetricsLogger(ml.MetricsLoggerOptions(log_dir=str(tmp_path), backend_kwargs={"custom_backend": [Recording]}))
  quiet.log("actor", "loss", 1.0, "train", 0)
  assert quiet._otel_meter is None                                           # off unless asked for
  lg.close(); quiet.close()


# ---- profiler -----------------------------------------------------------------------------------------
@pytest.fixture
def stub_tracing(monkeypatch):
  calls = []
  monkeypatch.setattr(prof.Profiler, "_start_trace", lambda self: calls.append(("start", self._output_path)))
  monkeypatch.setattr(prof.Profiler, "_stop_trace", lambda self: calls.append(("stop", self._output_path)))
  monkeypatch.setattr(prof.Profiler, "_is_active", False)
  monkeypatch.delenv("RANK", raising=False)
  return calls


def test_the_profile_window_starts_after_the_skipped_steps_and_is_capped_by_max_step(stub_tracing):
  opts = prof.ProfilerOptions(log_dir="/tmp/p", skip_first_n_steps=2, profiler_steps=3)
  p = prof.Profiler(initial_step=10, max_step=None, profiler_options=opts)
  assert (p._first_profile_step, p._last_profile_step) == (12, 15)
  for step in range(10, 18):
    p.maybe_activate(step)
    p.maybe_deactivate(step)
  assert stub_tracing == [("start", "/tmp/p"), ("stop", "/tmp/p")] and not prof.Profiler._is_active
  capped = prof.Profiler(initial_step=0, max_step=4, profiler_options=opts)
  assert (capped._first_profile_step, capped._last_profile_step) == (2, 4)
  with pytest.raises(ValueError, match="cannot be greater than the last profile step"):
    prof.Profiler(initial_step=0, max_step=2, profiler_options=opts)


def test_profiling_is_off_without_options_and_on_other_ranks(stub_tracing, monkeypatch):
  idle = prof.Profiler(0, None, None)
  idle.maybe_activate(0); idle.maybe_deactivate(0)
  monkeypatch.setenv("RANK", "3")
  other = prof.Profiler(0, None, prof.ProfilerOptions(log_dir="/tmp/p", skip_first_n_steps=0, profiler_steps=1))
  other.maybe_activate(0); other.maybe_deactivate(1)
  assert stub_tracing == []


def test_only_one_profiler_is_active_in_a_process(stub_tracing, caplog):
  a = prof.Profiler(0, None, prof.ProfilerOptions(log_dir="/tmp/a", skip_first_n_steps=0, profiler_steps=5))
  b = prof.Profiler(0, None, prof.ProfilerOptions(log_dir="/tmp/b", skip_first_n_steps=1, profiler_steps=2))
  a.maybe_activate(0)
  with caplog.at_level("WARNING"):
    b.maybe_activate(1)                                            # a is still tracing
  assert "already active" in caplog.text
  b.maybe_deactivate(3)                                            # b never started: it must not stop a's trace
  assert stub_tracing == [("start", "/tmp/a")] and prof.Profiler._is_active
  a.maybe_deactivate(5)
  assert stub_tracing[-1] == ("stop", "/tmp/a") and not prof.Profiler._is_active


def test_a_real_trace_is_written(tmp_path, monkeypatch):
  monkeypatch.delenv("RANK", raising=False)
  monkeypatch.setattr(prof.Profiler, "_is_active", False)
  p = prof.Profiler(0, None, prof.ProfilerOptions(log_dir=str(tmp_path), skip_first_n_steps=0, profiler_steps=1,
                                                  host_tracer_level=1, python_tracer_level=0))
  p.maybe_activate(0)
  torch.ones(8, 8) @ torch.ones(8, 8)
  p.maybe_deactivate(1)
  assert any(f.endswith(".json") or f.endswith(".json.gz") for f in os.listdir(tmp_path))
