"""ctypes binding of libaether_sort.so (the C ABI in include/aether_sort.h).

The binding follows the reference's own ctypes loader for its native library
(project_aether/src/custom_kernels/cuda/tma_collide.py:67-108): raw device
pointers, the stream as void*, an int status that is raised as RuntimeError.
There is no fallback: if the library is missing or fails to load, importing a
symbol from it raises.
"""

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(_PKG, 'libaether_sort.so')


class AetherGrid(ctypes.Structure):
    _fields_ = [('x0', ctypes.c_float), ('y0', ctypes.c_float), ('z0', ctypes.c_float),
                ('inv_dx', ctypes.c_float), ('inv_dy', ctypes.c_float),
                ('inv_dz', ctypes.c_float),
                ('nx', ctypes.c_int32), ('ny', ctypes.c_int32), ('nz', ctypes.c_int32),
                ('ix_offset', ctypes.c_int32), ('nx_local', ctypes.c_int32)]


_P = ctypes.c_void_p
_I64 = ctypes.c_int64
_SIGNATURES = {
    'AetherSortAbiVersion': (ctypes.c_int, []),
    'AetherSortWorkspaceBytes': (ctypes.c_size_t, [_I64, _I64, ctypes.c_int]),
    'AetherSortBucketPlan': (ctypes.c_int, [_I64, _I64, ctypes.POINTER(ctypes.c_int32),
                                            ctypes.POINTER(ctypes.c_int64),
                                            ctypes.POINTER(ctypes.c_int32)]),
    'AetherSortSetSmallShapeBucketLimit': (ctypes.c_int, [_I64]),
    'AetherSortSetChainedLaunches': (ctypes.c_int, [ctypes.c_int32]),
    'AetherSortParticlesByCell': (ctypes.c_int, [_P, _P, _P, _I64, ctypes.POINTER(AetherGrid),
                                                 ctypes.c_uint64, _P, _P, _P, _P, _P,
                                                 ctypes.c_size_t, _P]),
    'AetherSortAndGatherParticles': (ctypes.c_int, [_P, _P, _P, _P, _I64, _I64,
                                                    ctypes.POINTER(AetherGrid), ctypes.c_uint64,
                                                    _P, _P, _P, _P, _P, _P, _P, _P, _I64,
                                                    ctypes.c_int, _P, ctypes.c_size_t, _P]),
    'AetherPushSortAndGatherParticles': (ctypes.c_int, [_P, _P, _P, _P, _I64, _I64, ctypes.c_float,
                                                        ctypes.POINTER(ctypes.c_float),
                                                        ctypes.POINTER(ctypes.c_float),
                                                        ctypes.POINTER(AetherGrid), ctypes.c_uint64,
                                                        _P, _P, _P, _P, _P, _P, _P, _P, _I64,
                                                        ctypes.c_int, _P, ctypes.c_size_t, _P]),
    'AetherGatherParticles': (ctypes.c_int, [_P, _I64, _P, _P, _P, _P, _I64, _P, _P, _P, _P,
                                             _I64, _P]),
    'AetherMakeKeys': (ctypes.c_int, [_P, _P, _P, _I64, ctypes.POINTER(AetherGrid),
                                      ctypes.c_uint64, _P, _P]),
    'AetherSortReadStatus': (ctypes.c_int, [_P, _P, ctypes.POINTER(ctypes.c_int32)]),
    'AetherSortReadUsedDigitPasses': (ctypes.c_int, [_P, _P, ctypes.POINTER(ctypes.c_int32)]),
    'AetherSlabPartitionWorkspaceBytes': (ctypes.c_size_t, [_I64, ctypes.c_int]),
    'AetherSlabPartition': (ctypes.c_int, [_P, _P, _P, _P, _I64, _I64, ctypes.POINTER(AetherGrid),
                                           ctypes.c_int, _P, _P, _P, _P, _P, _P, _P, _P,
                                           ctypes.c_size_t, _P]),
    'AetherSlabExchangeCount': (ctypes.c_int, [_P, _I64, ctypes.POINTER(AetherGrid), ctypes.c_int,
                                               _P, _P, ctypes.c_size_t, _P]),
    'AetherSlabExchangeScatter': (ctypes.c_int, [_P, _P, _P, _P, _I64, _I64,
                                                 ctypes.POINTER(AetherGrid), ctypes.c_int,
                                                 ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
                                                 _I64, _P, _P, _P, ctypes.c_size_t, _P]),
    'AetherSlabExchangeCountMoved': (ctypes.c_int, [_P, _P, _I64, ctypes.c_float,
                                                    ctypes.POINTER(ctypes.c_float),
                                                    ctypes.POINTER(ctypes.c_float),
                                                    ctypes.POINTER(AetherGrid), ctypes.c_int, _P, _P,
                                                    ctypes.c_size_t, _P]),
    'AetherSlabExchangeScatterMoved': (ctypes.c_int, [_P, _P, _P, _P, _I64, _I64, ctypes.c_float,
                                                      ctypes.POINTER(ctypes.c_float),
                                                      ctypes.POINTER(ctypes.c_float),
                                                      ctypes.POINTER(AetherGrid), ctypes.c_int,
                                                      ctypes.c_int, ctypes.POINTER(ctypes.c_void_p),
                                                      _I64, _P, _P, _P, ctypes.c_size_t, _P]),
    'AetherSlabExchangeSliceCounts': (ctypes.c_int, [_I64, ctypes.c_int, ctypes.c_int, _P, _P,
                                                     ctypes.c_size_t, _P]),
    'AetherSlabSegmentsBytes': (ctypes.c_size_t, []),
    'AetherSlabExchangeSetResidentBlocks': (ctypes.c_int, [ctypes.c_int]),
    'AetherSlabExchangePrepare': (ctypes.c_int, [_P, ctypes.c_int, ctypes.c_int, ctypes.c_int, _P,
                                                 _P, _P]),
    'AetherSlabExchangeScatterSliced': (ctypes.c_int, [_P, _P, _P, _P, _I64, _I64, ctypes.c_float,
                                                       ctypes.POINTER(ctypes.c_float),
                                                       ctypes.POINTER(ctypes.c_float),
                                                       ctypes.POINTER(AetherGrid), ctypes.c_int,
                                                       ctypes.c_int,
                                                       ctypes.POINTER(ctypes.c_void_p), _I64, _P,
                                                       _P, ctypes.c_int, ctypes.c_int,
                                                       ctypes.c_uint32,
                                                       ctypes.POINTER(ctypes.c_void_p), _P,
                                                       ctypes.c_size_t, _P]),
    'AetherSlabExchangeSignal': (ctypes.c_int, [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                                ctypes.c_uint32, ctypes.POINTER(ctypes.c_void_p),
                                                _P]),
    'AetherSlabExchangeCopy': (ctypes.c_int, [_P, _P, ctypes.c_size_t, ctypes.c_int,
                                              ctypes.c_size_t, _P]),
    'AetherSlabExchangeWait': (ctypes.c_int, [_P, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                              ctypes.c_uint32, ctypes.c_uint32, _P, _P]),
    'AetherSortSlicedWorkspaceBytes': (ctypes.c_size_t, [_I64, _I64, _I64, ctypes.c_int]),
    'AetherSortSlicedBegin': (ctypes.c_int, [_I64, _I64, ctypes.POINTER(AetherGrid), ctypes.c_int,
                                             _P, ctypes.c_size_t, _P]),
    'AetherSortSlicedSlice': (ctypes.c_int, [_P, _P, _P, _P, _I64, _I64, _I64,
                                             ctypes.POINTER(AetherGrid), ctypes.c_uint64, _P,
                                             ctypes.c_int, ctypes.c_int, _P, ctypes.c_size_t, _P]),
    'AetherSortSlicedFinish': (ctypes.c_int, [_I64, _I64, ctypes.POINTER(AetherGrid), _P,
                                              ctypes.c_int, _P, _P, _P, _P, _P, _P, _P, _P, _I64,
                                              _P, ctypes.c_size_t, _P]),
    'AetherParticlePush': (ctypes.c_int, [_P, _P, _P, _P, _P, _P, _I64, ctypes.c_float,
                                          ctypes.POINTER(ctypes.c_float),
                                          ctypes.POINTER(ctypes.c_float), _P]),
    'AetherDsmcCollideTma': (ctypes.c_int, [_P] * 4 + [ctypes.c_int] * 3 + [ctypes.c_float] * 3 +
                             [ctypes.c_uint64] * 2 + [_P]),
    'AetherSortStaticMaxParticles': (ctypes.c_int64, []),
    'AetherSortParticlesByCellStatic': (ctypes.c_int, [_P, _P, _P, _I64,
                                                       ctypes.POINTER(AetherGrid),
                                                       ctypes.c_uint64, _P, _P, _P, _P, _P]),
    'AetherSortStaticReadStatus': (ctypes.c_int, [_P, ctypes.POINTER(ctypes.c_int32)]),
    'AetherSortStaticReadUsedDigitPasses': (ctypes.c_int, [_P, ctypes.POINTER(ctypes.c_int32)]),
    'AetherSortProbeLookbackWorkspaceBytes': (ctypes.c_size_t, []),
    'AetherSortProbeLookbackGiveUp': (ctypes.c_int, [_P, ctypes.c_size_t, ctypes.c_uint32, _P]),
    'AetherSortSetStageTiming': (ctypes.c_int, [ctypes.c_int]),
    'AetherSortStageCount': (ctypes.c_int, []),
    'AetherSortStageName': (ctypes.c_char_p, [ctypes.c_int]),
    'AetherSortReadStageTimes': (ctypes.c_int, [ctypes.POINTER(ctypes.c_float), ctypes.c_int]),
    'AetherSortKernelLaunches': (ctypes.c_uint64, []),
}

_library = None


def exported_symbols():
    """Names the header declares; every one must resolve in the library."""
    return tuple(_SIGNATURES)


def load_library(path: str | None = None) -> ctypes.CDLL:
    """Loads the CUDA library and declares the C ABI.

    The path is, in this order: the argument, the environment variable
    AETHER_SORT_LIBRARY, the library built in the package folder.

    Raises:
      OSError: if the library is not built or cannot be loaded.
    """
    global _library
    if _library is not None and path is None:
        return _library
    lib_path = path or os.environ.get('AETHER_SORT_LIBRARY') or LIBRARY_PATH
    if not os.path.exists(lib_path):
        raise OSError(f'{lib_path} is not built; run `python -m project_aether_b200.build`')
    library = ctypes.CDLL(lib_path)
    for name, (restype, argtypes) in _SIGNATURES.items():
        fn = getattr(library, name)
        fn.restype = restype
        fn.argtypes = argtypes
    if path is None:
        _library = library
    return library


def check(status: int, what: str) -> None:
    """Raises RuntimeError for a nonzero cudaError_t, as tma_collide.py:106-108 does."""
    if status != 0:
        raise RuntimeError(f'{what} failed with cudaError {status}')
