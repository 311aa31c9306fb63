"""`ClKernel` (user-written kernels): the example of the reference's README and
src/test/test_userkernel.lua with its known answer, tensor-info access, helper functions,
local memory with a barrier, and the argument errors of src/UserKernel.cpp.
"""
import numpy as np
import pytest

from tests.util import rng_uniform

ADD3 = """
   int linearId = get_global_id(0);
   if(linearId < nElements) {
     output_data[linearId] = input_data[linearId] + 3.0f;
   }
"""
ADD3_SPEC = {"input": {"nElements": "int", "input": "torch.ClTensor"}, "output": {"output": "torch.ClTensor"}, "src": ADD3}


# ---- argument checking: no GPU needed (raised before anything is compiled) --------------------

def test_spec_errors_follow_the_reference():
    import cltorch_b200 as cl
    with pytest.raises(cl.ClError, match="should be a table"):
        cl.ClKernel("src")
    with pytest.raises(cl.ClError, match="Missing parameter src, or was empty"):
        cl.ClKernel({"input": {"n": "int"}})
    with pytest.raises(cl.ClError, match="Unrecognized typename double"):
        cl.ClKernel({"input": {"n": "double"}, "src": ADD3})
    with pytest.raises(cl.ClError, match="ints can only be input parameters"):
        cl.ClKernel({"output": {"n": "int"}, "src": ADD3})
    with pytest.raises(cl.ClError, match="floats can only be input parameters"):
        cl.ClKernel({"inout": {"v": "float"}, "src": ADD3})
    with pytest.raises(cl.ClError, match="Parameter sauce not recognized"):
        cl.ClKernel({"sauce": "x", "src": ADD3})


# ---- on the GPU ------------------------------------------------------------------------------

@pytest.mark.gpu
def test_reference_example_known_answer():
    import cltorch_b200 as cl
    k = cl.ClKernel(ADD3_SPEC)
    x = cl.ClTensor(np.array([3, 5, 2], np.float32))
    y = cl.ClTensor(np.array([6, 4, 2], np.float32))
    k.run({"nElements": 3, "input": x, "output": y}, {"numWorkgroups": 10, "workgroupSize": 32})
    assert np.array_equal(y.float(), [6, 8, 5])                     # src/test/test_userkernel.lua
    assert np.array_equal(x.float(), [3, 5, 2])
    y2 = cl.ClTensor(3).fill(0)
    k.run({"nElements": 3, "input": x, "output": y2})               # default geometry, README.md:165
    assert np.array_equal(y2.float(), [6, 8, 5])
    assert k.getRawKernel() == ADD3
    rendered = k.getRenderedKernel()
    assert "typedef struct THClTensorInfoCl" in rendered and "user_kernel(" in rendered and ADD3 in rendered
    assert "input_info" in rendered and "float* output_data" in rendered and "int nElements" in rendered


@pytest.mark.gpu
def test_default_geometry_covers_a_large_output():
    import cltorch_b200 as cl
    n = 1_000_003
    a = rng_uniform(71, (n,))
    x, y = cl.ClTensor(a), cl.ClTensor(n).fill(-1)
    cl.ClKernel(ADD3_SPEC).run({"nElements": n, "input": x, "output": y})
    assert np.array_equal(y.float(), a + np.float32(3.0))


@pytest.mark.gpu
def test_tensor_info_gives_sizes_strides_and_offset():
    import cltorch_b200 as cl
    a = rng_uniform(72, (40, 50))
    base = cl.ClTensor(a)
    view = base.narrow(1, 6, 20).t()                                # 50 x 20, strides (1, 50), offset 5 * 50
    out = cl.ClTensor(50, 20).fill(0)
    k = cl.ClKernel({"name": "gather_view", "input": {"v": "ClTensor"}, "output": {"o": "ClTensor"}, "src": """
      int id = get_global_id(0);
      int rows = v_info->sizes[0], cols = v_info->sizes[1];
      if (id < rows * cols && v_info->dims == 2) {
        int r = id / cols, c = id % cols;
        o_data[o_info->offset + r * o_info->strides[0] + c * o_info->strides[1]] =
            v_data[v_info->offset + r * v_info->strides[0] + c * v_info->strides[1]];
      }
    """})
    k.run({"v": view, "o": out})
    assert "gather_view(" in k.getRenderedKernel()
    assert np.array_equal(out.float(), a[5:25].T)


@pytest.mark.gpu
def test_helper_functions_float_arguments_inout_and_local_memory():
    import cltorch_b200 as cl
    n = 64 * 37
    a = rng_uniform(73, (n,), -1, 1)
    t = cl.ClTensor(a)
    k = cl.ClKernel({
        "inout": {"data": "torch.ClTensor"}, "input": {"scale": "float", "n": "int"},
        "funcs": "float scaled(float v, float s) { return mad(v, s, 1.0f); }",
        "src": """
          local float buf[64];
          int lid = get_local_id(0), gid = get_global_id(0);
          buf[lid] = gid < n ? data_data[gid] : 0.0f;
          barrier(CLK_LOCAL_MEM_FENCE);
          // every work-group writes its 64 values back in reverse order
          int src = get_local_size(0) - 1 - lid;
          if (gid < n) data_data[gid] = scaled(buf[src], scale);
        """})
    k.run({"data": t, "scale": 2.5, "n": n})
    want = (a.reshape(-1, 64)[:, ::-1] * np.float32(2.5) + np.float32(1.0)).reshape(-1)
    assert np.allclose(t.float(), want, rtol=1e-6, atol=1e-6)


@pytest.mark.gpu
def test_opencl_qualifiers_in_helper_functions():
    """OpenCL spellings that helper functions of existing ClKernel sources use: a `local` pointer parameter,
    a `constant` table, the `kernel` word and mem_fence."""
    import cltorch_b200 as cl
    n = 64 * 5
    a = rng_uniform(74, (n,), -1, 1)
    t = cl.ClTensor(a)
    k = cl.ClKernel({
        "inout": {"data": "torch.ClTensor"}, "input": {"n": "int"},
        "funcs": """
          constant float weights[2] = {2.0f, 0.5f};
          float pick(local float* buf, int i) { return buf[i] * weights[i & 1]; }
        """,
        "src": """
          local float buf[64];
          int lid = get_local_id(0), gid = get_global_id(0);
          buf[lid] = gid < n ? data_data[gid] : 0.0f;
          mem_fence(CLK_LOCAL_MEM_FENCE);
          barrier(CLK_LOCAL_MEM_FENCE);
          if (gid < n) data_data[gid] = pick(buf, lid ^ 1);
        """})
    k.run({"data": t, "n": n})
    src = a.reshape(-1, 2)[:, ::-1].reshape(-1)               # neighbour within each pair
    w = np.where(np.arange(n) % 2 == 0, np.float32(0.5), np.float32(2.0))   # weight of the neighbour's slot
    assert np.array_equal(t.float(), (src * w).astype(np.float32))


@pytest.mark.gpu
def test_run_and_compile_errors():
    import cltorch_b200 as cl
    x = cl.ClTensor(np.zeros(4, np.float32))
    with pytest.raises(cl.ClError, match="Failed to create kernel"):
        cl.ClKernel({"output": {"o": "ClTensor"}, "src": "this is not C;"})
    k = cl.ClKernel({"input": {"i": "ClTensor", "n": "int"}, "src": "int id = get_global_id(0); (void)id;"})
    with pytest.raises(cl.ClError, match="Must provide at least one output, or inout, ClTensor"):
        k.run({"i": x, "n": 4})
    k2 = cl.ClKernel(ADD3_SPEC)
    with pytest.raises(cl.ClError, match="option colour not recognized"):
        k2.run({"nElements": 4, "input": x, "output": x}, {"colour": 3})
    with pytest.raises(cl.ClError, match="nElements is missing"):
        k2.run({"input": x, "output": x})
    with pytest.raises(cl.ClError, match="no data"):
        k2.run({"nElements": 4, "input": cl.ClTensor(), "output": x})
    with pytest.raises(cl.ClError, match="workgroupSize 4096 out of range"):
        k2.run({"nElements": 4, "input": x, "output": x}, {"workgroupSize": 4096})
