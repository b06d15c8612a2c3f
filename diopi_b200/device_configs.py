# Per-backend case filter for the reference's conformance harness: copy this file to impl/b200/device_configs.py of a
# DIOPI checkout and run the harness with --impl_folder pointing there. The harness imports `device_configs` from that
# folder (diopi_test/python/conformance/gen_case.py:39-49) and drops the marked parameter values
# (collect_case.py:35-102); `Skip` is the harness's own marker class (diopi_test/python/conformance/skip.py).
# Data only. The single thing this backend leaves unimplemented on its path is the interleaved rotary form, which the
# reference's CUDA backend also refuses (impl/torch/functions/functions_ext.cpp:45-48): diopiRotaryEmbedding returns
# diopiNoImplement for it.
from skip import Skip

device_configs = {
    'rotary_emb': dict(
        name=['rotary_emb'],
        para=dict(
            interleaved=[Skip(True)],
        ),
    ),

    'rotary_emb_empty_tensor': dict(
        name=['rotary_emb'],
        para=dict(
            interleaved=[Skip(True)],
        ),
    ),
}
