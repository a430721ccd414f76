"""The build refuses register spills in the kernels that keep tensor-memory loads in flight."""

from oops_b200.csrc.build import NO_SPILL_KERNELS, _spilling_entries

LOG = """ptxas info    : Compiling entry function '_ZN7oops_ta19ta_bwd_fused_kernelI13__nv_bfloat16Lb1EEEvNS_7FParamsE' for 'sm_100a'
ptxas info    : Function properties for _ZN7oops_ta19ta_bwd_fused_kernelI13__nv_bfloat16Lb1EEEvNS_7FParamsE
    8 bytes stack frame, 4 bytes spill stores, 4 bytes spill loads
ptxas info    : Used 96 registers, used 2 barriers, 8 bytes cumulative stack size
ptxas info    : Compiling entry function '_ZN7oops_ta13ta_fwd_kernelI6__halfLb1ELb1EEEvNS_9FwdParamsE' for 'sm_100a'
ptxas info    : Function properties for _ZN7oops_ta13ta_fwd_kernelI6__halfLb1ELb1EEEvNS_9FwdParamsE
    40 bytes stack frame, 44 bytes spill stores, 52 bytes spill loads
ptxas info    : Compiling entry function '_ZN7oops_ta19ta_bwd_dbias_kernelI6__halfEEvNS_8DbParamsE' for 'sm_100a'
ptxas info    : Function properties for _ZN7oops_ta19ta_bwd_dbias_kernelI6__halfEEvNS_8DbParamsE
    0 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads
"""


def test_guard_names_only_the_guarded_kernels_that_spill():
    found = _spilling_entries(LOG, NO_SPILL_KERNELS)
    assert len(found) == 1 and "ta_bwd_fused_kernel" in found[0] and "4 bytes" in found[0]
    assert _spilling_entries(LOG.replace("4 bytes spill stores", "0 bytes spill stores"), NO_SPILL_KERNELS) == []
