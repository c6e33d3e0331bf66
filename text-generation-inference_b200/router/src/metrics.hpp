// Prometheus metrics registry with the metric names and bucket layout of the reference router
// (router/src/server.rs:1937-2112; docs/source/reference/metrics.md): counters, gauges and
// histograms keyed by name + labels, rendered in the text exposition format at /metrics.
#pragma once
#include <cmath>
#include <map>
#include <mutex>
#include <sstream>
#include <string>
#include <utility>
#include <vector>

namespace sched {

using Labels = std::vector<std::pair<std::string, std::string>>;

struct Metrics {
  Metrics(double max_input_tokens = 4096, double max_total_tokens = 8192, double max_batch = 1024) {
    // durations: 35 geometric buckets from 0.15 ms with ratio 1.5
    double v = 0.00015;
    for (int i = 0; i < 35; ++i) {
      duration_buckets.push_back(v);
      v *= 1.5;
    }
    for (int i = 1; i <= 100; ++i) {
      input_buckets.push_back(max_input_tokens / 100.0 * i);
      total_buckets.push_back(max_total_tokens / 100.0 * i);
    }
    for (double b = 1; b <= max_batch; b *= 2) batch_buckets.push_back(b);
  }

  void counter_inc(const std::string& name, const Labels& labels = {}, double by = 1.0) {
    std::lock_guard<std::mutex> g(m_);
    counters_[key(name, labels)] += by;
  }
  void gauge_set(const std::string& name, double v) {
    std::lock_guard<std::mutex> g(m_);
    gauges_[name] = v;
  }
  void observe(const std::string& name, double seconds, const Labels& labels = {}) {
    observe_in(name, seconds, labels, duration_buckets);
  }
  void histogram_value(const std::string& name, double v) {
    const auto& b = name.find("input_length") != std::string::npos
                        ? input_buckets
                        : (name.find("batch") != std::string::npos ? batch_buckets : total_buckets);
    observe_in(name, v, {}, b);
  }

  std::string render() {
    std::lock_guard<std::mutex> g(m_);
    std::ostringstream o;
    for (auto& kv : counters_) o << kv.first << " " << kv.second << "\n";
    for (auto& kv : gauges_) o << kv.first << " " << kv.second << "\n";
    for (auto& kv : hists_) {
      const Hist& h = kv.second;
      const std::string base = h.name;
      for (size_t i = 0; i < h.bounds->size(); ++i)
        o << base << "_bucket{" << h.labels << (h.labels.empty() ? "" : ",") << "le=\"" << (*h.bounds)[i] << "\"} "
          << h.counts[i] << "\n";
      o << base << "_bucket{" << h.labels << (h.labels.empty() ? "" : ",") << "le=\"+Inf\"} " << h.count << "\n";
      o << base << "_sum" << (h.labels.empty() ? "" : "{" + h.labels + "}") << " " << h.sum << "\n";
      o << base << "_count" << (h.labels.empty() ? "" : "{" + h.labels + "}") << " " << h.count << "\n";
    }
    return o.str();
  }

  std::vector<double> duration_buckets, input_buckets, total_buckets, batch_buckets;

 private:
  struct Hist {
    std::string name, labels;
    const std::vector<double>* bounds = nullptr;
    std::vector<unsigned long long> counts;
    unsigned long long count = 0;
    double sum = 0;
  };
  static std::string label_str(const Labels& labels) {
    std::string s;
    for (size_t i = 0; i < labels.size(); ++i) {
      if (i) s += ",";
      s += labels[i].first + "=\"" + labels[i].second + "\"";
    }
    return s;
  }
  static std::string key(const std::string& name, const Labels& labels) {
    return labels.empty() ? name : name + "{" + label_str(labels) + "}";
  }
  void observe_in(const std::string& name, double v, const Labels& labels, const std::vector<double>& bounds) {
    std::lock_guard<std::mutex> g(m_);
    Hist& h = hists_[key(name, labels)];
    if (h.bounds == nullptr) {
      h.name = name;
      h.labels = label_str(labels);
      h.bounds = &bounds;
      h.counts.assign(bounds.size(), 0);
    }
    for (size_t i = 0; i < bounds.size(); ++i)
      if (v <= bounds[i]) ++h.counts[i];
    ++h.count;
    h.sum += v;
  }
  std::mutex m_;
  std::map<std::string, double> counters_, gauges_;
  std::map<std::string, Hist> hists_;
};

}  // namespace sched
