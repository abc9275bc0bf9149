"""Device discovery without a GPU: the second pass, the device environment and the attention predicate are driven with
fabricated devices and a fake probe child (the reference tests discovery the same way, discover/runner_test.go)."""
from ollama_b200.discover import devices as D

GiB = 1 << 30


def dev(i, uuid=False, major=10):
    return D.DeviceInfo(id=f"GPU-{i:08d}-aaaa-bbbb" if uuid else f"GPU-{i}", index=i, name="B200", compute_major=major, total_memory=180 * GiB, free_memory=170 * GiB)


def test_second_pass_keeps_only_devices_whose_child_answered():
    seen = []

    def child(cmd, env, timeout):
        seen.append((cmd[-1], env["CUDA_VISIBLE_DEVICES"], env["CUDA_DEVICE_ORDER"]))
        which = env["CUDA_VISIBLE_DEVICES"]
        if which == "1":
            return None                                  # crashed or hung
        if which == "2":
            return {"ok": False, "error": "device arithmetic is wrong"}
        return {"ok": True, "free_memory": 100 * GiB}

    out = D.validate_devices([dev(0), dev(1), dev(2), dev(3)], run_child=child, base_env={})
    assert [d.index for d in out] == [0, 3] and all(d.free_memory == 100 * GiB for d in out)
    assert sorted(s[1] for s in seen) == ["0", "1", "2", "3"] and all(s[0] == "--validate" and s[2] == "PCI_BUS_ID" for s in seen)
    assert D.validate_devices([], run_child=child) == []


def test_device_environment():
    env = D.devices_env([dev(2, uuid=True), dev(0, uuid=True)], base={"PATH": "/bin"})
    assert env["CUDA_VISIBLE_DEVICES"] == "GPU-00000002-aaaa-bbbb,GPU-00000000-aaaa-bbbb" and env["PATH"] == "/bin"
    assert D.devices_env([], base={})["CUDA_VISIBLE_DEVICES"] == "-1"
    # indices count within the devices already visible to this process
    assert D.devices_env([dev(1)], base={"CUDA_VISIBLE_DEVICES": "4,6"})["CUDA_VISIBLE_DEVICES"] == "6"
    assert D.devices_env([dev(1)], base={})["CUDA_VISIBLE_DEVICES"] == "1"


def test_filters_and_predicates():
    old, igpu = dev(1, major=9), dev(2)
    igpu.integrated = True
    assert [d.index for d in D.filter_devices([dev(0), old, igpu])] == [0]
    assert D.flash_attention_supported([dev(0), dev(1)]) and D.flash_attention_supported([]) and not D.flash_attention_supported([dev(0), old])


def test_probe_child_reports_instead_of_raising(capsys):
    from ollama_b200.discover import probe
    assert probe.main(["--validate"]) == 0
    import json
    ans = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert ans["ok"] is False and ans["error"]              # no CUDA device here
    assert probe.main([]) == 0 and json.loads(capsys.readouterr().out.strip().splitlines()[-1])["devices"] == []
