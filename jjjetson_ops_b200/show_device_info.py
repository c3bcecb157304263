"""Prints what the library knows about a GPU, in the line format of the reference's
``tools/show_device_info.cu`` (``[DeviceHwInfo] key: value``, include/device_hw_info.cuh:252-350), with
the rows the reference's tables lack for compute capability 10.0: int8 / bf16 tensor peaks, the HBM
peak and the int8 ridge point.

    python -m jjjetson_ops_b200.show_device_info [device_id]
"""
import sys

from . import capi


def format_lines(info: dict) -> list:
    gb = 1e9
    rows = [
        ("device_id", "%d" % info["device_id"]),
        ("name", info["name"]),
        ("compute_capability", "%d.%d" % (info["cc_major"], info["cc_minor"])),
        ("sm_count", "%d" % info["sm_count"]),
        ("sm_clock_ghz", "%.6f" % (info["sm_clock_khz"] / 1e6)),
        ("mem_clock_ghz", "%.6f" % (info["mem_clock_khz"] / 1e6)),
        ("mem_bus_width_bits", "%d" % info["mem_bus_width_bits"]),
        ("total_global_mem_gbytes", "%.6f" % (info["global_mem_bytes"] / gb)),
        ("l2_cache_bytes", "%d" % info["l2_bytes"]),
        ("shared_mem_per_block_optin_kibytes", "%.6f" % (info["smem_per_block_optin"] / 1024.0)),
        ("shared_mem_per_multiprocessor_kibytes", "%.6f" % (info["smem_per_sm"] / 1024.0)),
        ("max_warps_per_multiprocessor", "%d" % info["max_warps_per_sm"]),
        ("warp_schedulers_per_sm", "%d" % info["warp_schedulers_per_sm"]),
        ("fp32_cores_per_sm (table)", "%d" % info["fp32_cores_per_sm"]),
        ("peak_dram_theoretical", "%.6f GB/s" % info["peak_dram_gbs"]),
        ("peak_fp32_tflops_theoretical", "%.6f" % info["peak_fp32_tflops"]),
        ("peak_tc_bf16_dense_tflops_nominal", "%.6f" % info["peak_bf16_dense_tflops"]),
        ("peak_tc_int8_dense_tops_nominal", "%.6f" % info["peak_int8_dense_tops"]),
        ("roofline_ridge_tc_int8_dense_vs_dram_ops_per_byte", "%.6f" % info["ridge_int8_ops_per_byte"]),
    ]
    return ["[DeviceHwInfo] %s: %s" % kv for kv in rows]


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    device = int(argv[0]) if argv else 0
    try:
        info = capi.query_device_hw_info(device)
    except capi.JqError as e:
        print("query_device_hw_info(%d) failed: %s" % (device, e), file=sys.stderr)
        return 1
    print("\n".join(format_lines(info)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
