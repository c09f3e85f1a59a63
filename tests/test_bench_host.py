"""Host-side pieces of bench.py that need no GPU: the parser that turns an ncu DRAM capture into profiles/dram_traffic.json
and the roofline arithmetic."""
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402

CSV = '''==PROF== Connected to process 1
"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"
"0","1","python","h","void b2vx::<unnamed>::gemm_i8_tc_kernel<0, 0>(CUtensorMap_st, GemmParams)","1","7","(640, 1, 1)","(148, 1, 1)","0","10.0","Command line profiler metrics","dram__bytes_read.sum","Mbyte","10.5"
"0","1","python","h","void b2vx::<unnamed>::gemm_i8_tc_kernel<0, 0>(CUtensorMap_st, GemmParams)","1","7","(640, 1, 1)","(148, 1, 1)","0","10.0","Command line profiler metrics","dram__bytes_write.sum","Kbyte","500"
"1","1","python","h","void b2vx::<unnamed>::gemm_i8_tc_kernel<0, 1>(CUtensorMap_st, GemmParams)","1","7","(640, 1, 1)","(148, 1, 1)","0","10.0","Command line profiler metrics","dram__bytes_read.sum","Mbyte","4"
"1","1","python","h","void b2vx::<unnamed>::gemm_i8_tc_kernel<0, 1>(CUtensorMap_st, GemmParams)","1","7","(640, 1, 1)","(148, 1, 1)","0","10.0","Command line profiler metrics","dram__bytes_write.sum","byte","0"
"2","1","python","h","void b2vx::pool_q16_kernel<0, 3>(const unsigned char *)","1","7","(256, 1, 1)","(784, 1, 1)","0","10.0","Command line profiler metrics","dram__bytes_read.sum","Mbyte","3"
"2","1","python","h","void b2vx::pool_q16_kernel<0, 3>(const unsigned char *)","1","7","(256, 1, 1)","(784, 1, 1)","0","10.0","Command line profiler metrics","dram__bytes_write.sum","Mbyte","1"
'''


class Args:
    pass


def test_traffic_record_sums_both_instantiations_of_the_dominant_kernel(tmp_path, monkeypatch, capsys):
    src = tmp_path / "dram.csv"
    src.write_text(CSV)
    out = tmp_path / "dram_traffic.json"
    monkeypatch.setattr(bench, "TRAFFIC_FILE", str(out))
    a = Args()
    a.traffic_from, a.workload, a.batch = str(src), "resnet50", 64
    assert bench.record_traffic(a) == 0
    rec = json.loads(out.read_text())["resnet50:64"]
    assert rec["kernel"] == "gemm_i8_tc_kernel" and rec["launches"] == 2
    assert rec["bytes"] == 10.5e6 + 500e3 + 4e6
    assert bench.dram_traffic("resnet50", 64)["bytes"] == rec["bytes"]
    assert bench.dram_traffic("resnet50", 8) is None


def test_roofline_picks_the_binding_limit():
    # above the ridge (ops per byte > peak ops / peak bytes): tensor-bound; below: memory-bound
    hbm, peak = 6500.0, 4000.0
    hi = bench.roofline_of({"ops": 4e12, "bytes": 1e9, "ms": 2.0}, hbm, peak)
    assert hi["bound"] == "tensor" and abs(hi["achieved"] - 2000.0) < 1e-6 and abs(hi["frac"] - 0.5) < 1e-9
    lo = bench.roofline_of({"ops": 1e9, "bytes": 6.5e9, "ms": 2.0}, hbm, peak)
    assert lo["bound"] == "hbm" and abs(lo["achieved"] - 3250.0) < 1e-6 and abs(lo["frac"] - 0.5) < 1e-9
