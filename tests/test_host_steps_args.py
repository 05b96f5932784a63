"""Argument checks of the host-buffer decode steps that run before any CUDA call, and the loud
failure without a device (no CPU fallback)."""

import ctypes

import pytest
import torch


def test_create_rejects_bad_arguments_before_touching_cuda(built_lib):
    lib = built_lib
    h = ctypes.c_void_p()
    assert lib.b200kv_host_steps_create(0, 4, 8, 2, 128, ctypes.byref(h)) == 1      # depth < 1
    assert lib.b200kv_host_steps_create(9, 4, 8, 2, 128, ctypes.byref(h)) == 1      # depth > 8
    assert lib.b200kv_host_steps_create(2, 0, 8, 2, 128, ctypes.byref(h)) == 1      # no batch
    assert lib.b200kv_host_steps_create(2, 4, 8, 3, 128, ctypes.byref(h)) == 1      # heads do not divide
    assert lib.b200kv_host_steps_create(2, 4, 8, 2, 128, None) == 1                 # nowhere to put the handle
    assert lib.b200kv_host_steps_create(2, 4, 8, 2, 64, ctypes.byref(h)) == 2       # head_dim not built
    assert lib.b200kv_host_steps_create(2, 4, 34, 2, 128, ctypes.byref(h)) == 2     # query group above 16
    assert not h.value


def test_null_handle_is_an_argument_error(built_lib):
    lib = built_lib
    assert lib.b200kv_host_steps_wait(None, 0) == 1
    assert lib.b200kv_host_steps_flush(None) == 1
    assert lib.b200kv_host_steps_reset(None) == 1
    assert lib.b200kv_host_steps_buffers(None, 0, 1, None, None, None, None, None, None) == 1
    assert lib.b200kv_host_steps_stream(None) is None
    lib.b200kv_host_steps_destroy(None)      # like free(NULL)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour without a CUDA device")
def test_without_a_device_the_constructor_raises(built_lib):
    from llama_lite_npu_b200.host_step import HostDecodeSteps

    with pytest.raises(Exception):
        HostDecodeSteps(4, 8, 2, 128, device=0)
    h = ctypes.c_void_p()
    assert built_lib.b200kv_host_steps_create(2, 4, 8, 2, 128, ctypes.byref(h)) == 5   # B200KV_ECUDA
    assert not h.value
