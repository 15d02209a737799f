"""The step profiler's bookkeeping: kernel names fall into families, zero-time (host-only) events are dropped and the
table is per step."""
from maxdiffusion_b200.utils import step_profile as SP


class _Event:

  def __init__(self, key, count, device_us):
    self.key, self.count, self.device_time_total = key, count, device_us


def test_kernel_names_map_to_families():
  assert SP.family("void mdb::flash::flash_fwd_kernel<128, 3>(Params)") == "attention forward"
  assert SP.family("mdb::flash::flash_bwd_dkv_kernel<128>") == "attention backward dK/dV"
  assert SP.family("mdb::conv::conv_igemm_kernel<2>") == "conv forward / input gradient"
  assert SP.family("mdb::conv::conv_wgrad_kernel") == "conv weight gradient"
  assert SP.family("ncclDevKernel_ReduceScatter_Sum_bf16_RING_LL") == "NCCL"
  assert SP.family("void at::native::vectorized_elementwise_kernel<4, ...>") == "PyTorch elementwise / copies"
  assert SP.family("something_new") == "other"


def test_summary_is_per_step_and_sorted_by_device_time():
  events = [_Event("mdb::flash::flash_fwd_kernel<128,3>", 4, 8000.0), _Event("mdb::conv::conv_igemm_kernel<2>", 10, 3000.0),
            _Event("mdb::conv::conv_igemm_kernel<1>", 2, 1000.0), _Event("aten::add", 5, 0.0)]
  assert SP.summarise(events, 2) == [("attention forward", 2, 4.0), ("conv forward / input gradient", 6, 2.0)]
