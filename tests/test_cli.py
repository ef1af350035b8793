"""flash-attn-benchmark: argument handling and FLOP counting on CPU, one timed run on a GPU."""
import json

import pytest
import torch

from flash_attention_v100 import cli


def test_flop_count_matches_the_workload_table():
    # B4 N4096 H32 D128 causal: 549.8 GFLOP forward, 2.5 times that backward
    fl = cli.attention_flops(4, 4096, 4096, 32, 128, True)
    assert fl["fwd"] == pytest.approx(549.8e9, rel=1e-3)
    assert fl["bwd"] == pytest.approx(2.5 * fl["fwd"])
    assert cli.attention_flops(8, 2048, 2048, 16, 64, False)["fwd"] == pytest.approx(137.4e9, rel=1e-3)


def test_device_info_keys():
    info = cli.get_device_info()
    for key in ("cuda_available", "cuda_device_count", "pytorch_version", "distributed_available",
                "distributed_initialized", "system"):
        assert key in info
    assert info["cuda_available"] == torch.cuda.is_available()


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour without a device")
def test_main_without_a_device_reports_and_fails(capsys):
    assert cli.main(["--steps", "1", "--warmup", "0"]) == 1
    assert "no CPU path" in capsys.readouterr().out
    with pytest.raises(RuntimeError):
        cli.run_benchmark(1, 128, 1, 64, torch.float16, False)


def test_bad_head_dim_is_rejected():
    with pytest.raises(SystemExit):
        cli.main(["--head-dim", "96"])


@pytest.mark.gpu
def test_main_json_on_gpu(capsys, device):
    rc = cli.main(["--batch", "2", "--seq-len", "512", "--heads", "4", "--head-dim", "64", "--dtype", "fp16",
                   "--no-causal", "--steps", "3", "--warmup", "1", "--json"])
    assert rc == 0
    res = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert res["shape"] == [2, 512, 4, 64] and res["fwd_ms"] > 0 and res["bwd_ms"] > 0
    assert res["fwd_bwd_tflops"] > 0


@pytest.mark.gpu
def test_sequence_parallel_mode_on_one_gpu(capsys, device, monkeypatch):
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    for k, v in (("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", str(port)), ("RANK", "0"), ("WORLD_SIZE", "1"),
                 ("LOCAL_RANK", "0")):
        monkeypatch.setenv(k, v)
    rc = cli.main(["--sequence-parallel", "zigzag", "--batch", "1", "--seq-len", "512", "--heads", "2",
                   "--head-dim", "64", "--steps", "2", "--warmup", "1", "--json"])
    assert rc == 0
    res = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert res["n_gpus"] == 1 and res["per_rank"] == 512 and res["layout"] == "zigzag"
    assert res["ms_per_step"] > 0 and res["fwd_bwd_tflops"] > 0
