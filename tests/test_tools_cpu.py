"""Stand-alone tools: the LD_PRELOAD CUDA API counter (against a fake runtime), the GSM8K evaluation
script and the QPS sweep of the serving benchmark (both against the CPU fake engine)."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(subprocess.run(["which", "gcc"], capture_output=True).returncode != 0, reason="needs gcc")
def test_cuda_api_counter_counts_calls_of_a_fake_runtime(tmp_path):
    shim = tmp_path / "libcounter.so"
    src = os.path.join(ROOT, "pegainfer_b200", "utils", "cuda_api_counter.c")
    subprocess.run(["gcc", "-O2", "-shared", "-fPIC", "-o", str(shim), src, "-ldl"], check=True)
    # a fake CUDA runtime and a program that calls it: no GPU, no real libcudart involved
    (tmp_path / "fake.c").write_text(
        "#include <stddef.h>\n int cudaMalloc(void** p, size_t n) { *p = (void*)16; return 0; }\n int cudaFree(void* p) { return 0; }\n"
        " int cudaGraphLaunch(void* g, void* s) { return 0; }\n int cudaMemcpyAsync(void* d, const void* s, size_t n, int k, void* st) { return 0; }\n")
    (tmp_path / "main.c").write_text(
        "#include <stddef.h>\n int cudaMalloc(void**, size_t); int cudaFree(void*); int cudaGraphLaunch(void*, void*); int cudaMemcpyAsync(void*, const void*, size_t, int, void*);\n"
        " int main() { void* p; for (int i = 0; i < 3; ++i) cudaMalloc(&p, 64); cudaFree(p); for (int i = 0; i < 7; ++i) { cudaMemcpyAsync(p, p, 4, 1, 0); cudaGraphLaunch(0, 0); } return 0; }\n")
    subprocess.run(["gcc", "-shared", "-fPIC", "-o", str(tmp_path / "libfakecudart.so"), str(tmp_path / "fake.c")], check=True)
    subprocess.run(["gcc", "-o", str(tmp_path / "prog"), str(tmp_path / "main.c"), f"-L{tmp_path}", "-lfakecudart", f"-Wl,-rpath,{tmp_path}"], check=True)
    out = tmp_path / "counts.txt"
    env = dict(os.environ, LD_PRELOAD=str(shim), PEGAINFER_API_COUNTER_OUT=str(out))
    subprocess.run([str(tmp_path / "prog")], check=True, env=env)
    counts = dict(line.split() for line in out.read_text().splitlines())
    assert counts["cudaMalloc"] == "3" and counts["cudaFree"] == "1" and counts["cudaGraphLaunch"] == "7" and counts["cudaMemcpyAsync"] == "7" and counts["cudaLaunchKernel"] == "0"
    # while the hold file exists nothing is counted
    hold = tmp_path / "hold"
    hold.write_text("")
    subprocess.run([str(tmp_path / "prog")], check=True, env=dict(env, PEGAINFER_API_COUNTER_RESET=str(hold)))
    assert dict(line.split() for line in out.read_text().splitlines())["cudaMalloc"] == "0"


def test_gsm8k_eval_extraction_and_http_loop(tmp_path):
    sys.path.insert(0, ROOT)
    import eval_gsm8k as e

    assert e.gold_answer("... so 5 + 7 = 12\n#### 1,234") == 1234
    assert e.extract_answer("<think>maybe 17</think>Therefore #### 42.0") == 42
    assert e.extract_answer("The answer is $3,000.50.") == 3000.5 and e.extract_answer("first 7 then 9") == 9 and e.extract_answer("no numbers") is None
    data = tmp_path / "d.jsonl"
    data.write_text("\n".join(json.dumps({"question": f"q{i}", "answer": f"work\n#### {i}"}) for i in range(4)))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "eval_gsm8k.py"), "--spawn", "sim", "--data", str(data), "--max-tokens", "4", "--out", str(tmp_path / "rec.jsonl")], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "GSM8K strict match:" in r.stdout and "failed requests: 0" in r.stdout, r.stdout + r.stderr
    recs = [json.loads(l) for l in (tmp_path / "rec.jsonl").read_text().splitlines()]
    assert len(recs) == 4 and all(x["error"] is None for x in recs)


def test_serving_bench_qps_sweep_against_sim_engine(tmp_path):
    out = tmp_path / "sweep.json"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench_serving.py"), "--spawn", "sim", "--num-prompts", "10", "--input-len", "16", "--output-len", "6", "--qps-sweep", "25,50", "--json", str(out)],
                       capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, r.stdout + r.stderr
    sweep = json.loads(out.read_text())["sweep"]
    assert [s["request_rate"] for s in sweep] == [25.0, 50.0] and all(s["completed"] == 10 and s["failed"] == 0 for s in sweep)
