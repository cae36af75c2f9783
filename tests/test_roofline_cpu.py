"""Bandwidth floor of a decode cycle from the model shapes."""
from smcsd_b200.models.config import preset
from smcsd_b200.utils.roofline import decode_cycle_floor, dense_weight_bytes, measured_peaks


def test_weight_bytes_of_the_headline_pair():
    t, d = preset("llama-3.1-8b"), preset("llama-3.2-1b")
    assert abs(dense_weight_bytes(t) / 1e9 - 15.0) < 0.1          # 7.5 G weights in bf16
    assert abs(dense_weight_bytes(d) / 1e9 - 2.47) < 0.05         # tied head counted once
    f = decode_cycle_floor(t, d, gamma=8, rows=8, context=512, shared_prompt=256, hbm_gbs=6453.0)
    # 15.0 + 8 x 2.47 GB of weights, a few hundred MB of cached keys and values: about 5.4 ms at 6453 GB/s
    assert 5.3 < f["floor_ms"] < 5.6 and f["weight_bytes"] > 30 * f["kv_bytes"]
    g = decode_cycle_floor(t, d, gamma=8, defer_bonus=False, rows=8, hbm_gbs=6453.0)
    assert g["weight_bytes"] - f["weight_bytes"] == dense_weight_bytes(d)


def test_peaks_record_or_fallback(tmp_path):
    p = tmp_path / "peaks.json"
    p.write_text('{"hbm_gbs": 6000.0, "bf16_tflops": 1500.0}')
    assert measured_peaks(str(p)) == (6000.0, 1500.0, "measured")
    assert measured_peaks(str(tmp_path / "absent.json")) == (6650.0, 1590.0, "fallback")
    assert decode_cycle_floor(preset("tiny-target"), preset("tiny-draft"), gamma=4, hbm_gbs=1000.0)["floor_ms"] > 0
