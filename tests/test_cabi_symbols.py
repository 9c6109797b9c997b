"""The C ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os

from insconv import cabi


def test_header_and_binding_agree():
    declared = cabi.declared_symbols()
    assert len(declared) >= 30
    assert set(declared) == set(cabi.PROTOTYPES)


def test_library_exports_every_declared_symbol():
    assert os.path.exists(cabi.LIB_PATH), "run python ins-conv_b200/build.py"
    lib = ctypes.CDLL(cabi.LIB_PATH)
    for name in cabi.declared_symbols():
        assert hasattr(lib, name), name


def test_no_compute_calls_needed_for_identification():
    lib = cabi.lib()
    assert b"sm_100a" in lib.scn_version()
    assert lib.scn_n_rulebook_bits() == 32
    assert lib.scn_last_error() is not None


def test_argument_errors_do_not_need_a_gpu():
    import pytest
    with pytest.raises(cabi.ScnError) as e:
        cabi.call("scn_metadata_clear", None, None)
    assert e.value.code == -1
    h = ctypes.c_void_p()
    cabi.call("scn_metadata_create", ctypes.byref(h))
    assert cabi.lib().scn_metadata_n_active(h, cabi.size3(64)) == -1
    with pytest.raises(cabi.ScnError) as e:
        cabi.call("scn_ssc_rulebook", h, cabi.size3(64), None, None, None)
    assert e.value.code == -5
    with pytest.raises(cabi.ScnError) as e:  # mode 1 is not part of the GPU grid path
        n = ctypes.c_int64()
        cabi.call("scn_input_layer_build", h, cabi.size3(64), None, 1, 0, 3, 0, 1, None, ctypes.byref(n))
    assert e.value.code == -6
    cabi.lib().scn_metadata_destroy(h)


def test_extension_module_exports_the_reference_operator_names():
    import sparseconvnet as scn
    for name in ["Metadata_3", "SubmanifoldConvolution_updateOutput", "Convolution_updateOutput",
                 "Deconvolution_updateOutput", "BatchNormalization_updateOutput", "NetworkInNetwork_updateOutput",
                 "InputLayer_updateOutput", "OutputLayer_updateOutput", "Incre_SubmanifoldConvolution_updateOutput",
                 "Incre_Convolution_updateOutput", "Incre_Deconvolution_updateOutput",
                 "Incre_BatchNormalization_updateOutput", "Incre_InputLayer_updateOutput",
                 "Incre_OutputLayer_updateOutput", "n_rulebook_bits", "SubmanifoldConvolution_backward"]:
        assert hasattr(scn.SCN, name), name
    assert scn.SCN.n_rulebook_bits() == 32
    import pytest
    with pytest.raises(RuntimeError):
        scn.SCN.SubmanifoldConvolution_backward()
    # label fusion classes and the whole method surface of the reference's Metadata class (pybind.cpp:13-45, 275-282)
    for cls, methods in (("Result_3", ["set", "query", "multiQuery", "clear", "update", "get_all_points_labels", "finalize"]),
                         ("ResultOfWeight", ["query", "multiQuery", "clear", "update", "get_all_points_labels", "finalize"]),
                         ("Metadata_3", ["clear", "setInputSpatialSize", "setNormalGuideScale", "batchAddSample",
                                         "setInputSpatialLocation", "setInputSpatialLocations", "getSpatialLocations",
                                         "createMetadataForDenseToSparse", "sparsifyMetadata", "appendMetadata",
                                         "sparsifyCompare", "addSampleFromThresholdedTensor", "generateRuleBooks3s2",
                                         "generateRuleBooks2s2", "compareSparseHelper"])):
        for name in methods:
            assert hasattr(getattr(scn.SCN, cls), name), (cls, name)
