"""The examples that need no GPU run as written and exit 0."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("script", ["examples/memory_pool/01_two_rank_dram_pool.py", "examples/memory_pool/02_copy_data_batch_and_register.py",
                                    "examples/memory_pool/04_extend_local_mem.py", "examples/memory_pool/05_observability/metrics_endpoint.py",
                                    "examples/memory_pool/06_enable_56bits_gva.py",
                                    "examples/transfer/transfer_engine.py", "examples/tensor_rtl/reshard_tp4_to_tp2.py",
                                    "examples/tensor_rtl/eplb_expert_migration.py", "examples/tensor_rtl/rl_train_to_infer_reshard.py"])
def test_example_runs(script):
    env = dict(os.environ, MF_DEVICE_BACKEND="none")
    env.pop("RANK", None)
    env.pop("WORLD_SIZE", None)
    r = subprocess.run([sys.executable, os.path.join(ROOT, script)], env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


def test_dashboard_and_scrape_config_refer_to_exported_metrics(tmp_path):
    """Every metric a panel of the Grafana dashboard queries is a family the exporter produces, the dashboard's variables are
    labels of the scrape configuration, and the latency panels use the histogram."""
    import json
    import re

    import yaml
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import hooks as H
    from memfabric_hybrid_b200.utils import metrics
    from memfabric_hybrid_b200.zbal import _capi as K
    d = os.path.join(ROOT, "examples/memory_pool/05_observability")
    dash = json.load(open(os.path.join(d, "grafana_dashboard.json")))
    prom = yaml.safe_load(open(os.path.join(d, "prometheus.yaml")))
    labels = set(prom["scrape_configs"][0]["static_configs"][0]["labels"])
    assert {"cluster", "node", "rank", "device_id"} <= labels and prom["scrape_configs"][0]["metrics_path"] == "/metrics"
    assert {v["name"] for v in dash["templating"]["list"]} - {"datasource"} <= labels

    class Pool:   # stands in for a BigMemory handle
        def copy_stats(self):
            return dict.fromkeys(("kernel_launches", "kernel_chunks", "engine_copies", "host_copies", "vm_copies", "coalesced"), 1)

        def local_mem_size(self, mem):
            return 1 << 20
    l = H.lib()
    assert l.mf_t_trace_start(str(tmp_path).encode(), 60_000) == 0
    try:
        l.mf_t_trace_hit(10, 0, 10)
        K.lib().zbal_simulate_init(0x7000_0000_0000, 64 << 20)
        metrics.register_pool("kv", Pool())
        text = metrics.render()
    finally:
        metrics.unregister_pool("kv")
        K.lib().zbal_sma_uninit(0)
        l.mf_t_trace_stop()
    exported = {line.split("{")[0].split(" ")[0] for line in text.splitlines() if line and not line.startswith("#")}
    used = set()
    for p in dash["panels"]:
        assert p["targets"], p["title"]
        for t in p["targets"]:
            used |= set(re.findall(r"\b((?:mf|zbal)_[a-z_]+)\b", t["expr"]))
    assert used and used <= exported, sorted(used - exported)
    assert any("histogram_quantile(0.99" in t["expr"] for p in dash["panels"] for t in p["targets"])
    assert len({p["id"] for p in dash["panels"]}) == len(dash["panels"]) == 8
