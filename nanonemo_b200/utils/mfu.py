"""Model FLOPs per token and MFU against a per-GPU peak.

FLOPs / token = 6 * N_matmul + 12 * n_layers * d_model * seq_len (PaLM appendix B; the tied head is
counted once as a matmul, attention over the full T x T square) — the reference's definition
(nanonemo/utils/mfu.py:1-31), 798,031,872 at the 114M shape and seq 1024. The peak tables keep the
reference's Turing/Ada entries and add B200: nominal dense figures, overridden by the pool's
measured cuBLAS bf16 throughput and copy bandwidth when MEASURED_PEAKS.json is present.
"""

from nanonemo_b200.models.config import ModelConfig


def matmul_params(cfg: ModelConfig) -> int:
    d, hd = cfg.d_model, cfg.head_dim
    q, kv = cfg.n_heads * hd, cfg.n_kv_heads * hd
    attn = d * (q + 2 * kv) + q * d
    mlp = 3 * d * cfg.d_ff
    return cfg.n_layers * (attn + mlp) + cfg.vocab_size * d


def flops_per_token(cfg: ModelConfig, seq_len: int) -> int:
    return 6 * matmul_params(cfg) + 12 * cfg.n_layers * cfg.n_heads * cfg.head_dim * seq_len


PEAK_TFLOPS = {
    "rtx 2070 super": {"fp16_tc": 28.3, "fp32": 7.07},
    "t4": {"fp16_tc": 65.0, "fp32": 8.1},
    "l4": {"fp16_tc": 121.0, "bf16_tc": 121.0, "fp32": 30.3},
    # B200 nominal dense (no 2:4 sparsity): bf16/fp16 2250, fp8 4500, tf32 1100.
    "b200": {"fp16_tc": 2250.0, "bf16_tc": 2250.0, "fp8_tc": 4500.0, "fp32": 80.0},
}
RATED_BOOST_MHZ = {"rtx 2070 super": 1380}
PEAK_GBPS = {"rtx 2070 super": 448.0, "t4": 320.0, "l4": 300.0, "b200": 7700.0}


def _lookup(table: dict, device_name: str):
    name = device_name.lower()
    for junk in ("nvidia", "geforce", "tesla", "laptop gpu"):
        name = name.replace(junk, "")
    name = " ".join(name.split())
    for key in sorted(table, key=len, reverse=True):
        if name == key or name.startswith(key + " "):
            return table[key]
    return None


def peak_tflops(device_name: str) -> dict | None:
    entry = _lookup(PEAK_TFLOPS, device_name)
    if entry is not None and "b200" in device_name.lower():
        from nanonemo_b200.utils.env import measured_peaks

        m = measured_peaks()
        if m:
            entry = dict(entry, bf16_measured=m.get("bf16_tflops"), bf16_measured_sustained=m.get("bf16_tflops_sustained"))
    return entry


def peak_gbps(device_name: str) -> float | None:
    if "b200" in device_name.lower():
        from nanonemo_b200.utils.env import measured_peaks

        m = measured_peaks()
        if m and m.get("hbm_gbs"):
            return float(m["hbm_gbs"])
    return _lookup(PEAK_GBPS, device_name)


def rated_boost_mhz(device_name: str) -> int | None:
    return _lookup(RATED_BOOST_MHZ, device_name)


def mfu(tokens_per_s: float, flops_per_tok: int, peak_tflops_value: float) -> float:
    return tokens_per_s * flops_per_tok / (peak_tflops_value * 1e12)
