// Compile check of the reference-side binding: the bodies a maintainer of OpenNN would put into
// opennn/normalization_layer_3d.cpp (:198-215 forward, :218-241 backward) to run Normalization3d on this library.
// The translation unit includes the reference's OWN headers with its CUDA path switched on (WITH_CUDA, opennn/pch.h:68-70)
// and defines the two `...Cuda` overrides that opennn/layer.h:348-358 declares, calling the C ABI of
// include/onn_b200.h with the members OpenNN's propagation structures hold.  It is compiled, never linked or run:
// if a signature, a member name or a type of either side moves, this file stops compiling.
//
// TEST INFRASTRUCTURE (built by `make -C oracle binding-check` into oracle/_ref/); no reference source is copied.
#define WITH_CUDA
#include "pch.h"
#include "normalization_layer_3d.h"

#include "onn_b200.h"

namespace opennn
{

static void check_onn_status(int status, const char* what)
{
    if(status != ONN_OK) throw runtime_error(string(what) + ": " + onn_status_string(status));
}

void Normalization3d::forward_propagate(unique_ptr<LayerForwardPropagationCuda>& forward_propagation, bool)
{
    Normalization3dForwardPropagationCuda* fp_cuda = static_cast<Normalization3dForwardPropagationCuda*>(forward_propagation.get());

    const int64_t rows = int64_t(fp_cuda->batch_size * sequence_length);
    const int64_t features = int64_t(get_embedding_dimension());

    // OpenNN computes on the legacy default stream (opennn/adaptive_moment_estimation.cpp:705): stream = nullptr
    check_onn_status(onn_layernorm_fwd(forward_propagation->inputs[0].data, nullptr,
                                       gammas_device.data, betas_device.data,
                                       fp_cuda->outputs.data, nullptr,
                                       fp_cuda->means_device.data, fp_cuda->inv_variances_device.data, nullptr,
                                       rows, features, static_cast<float>(EPSILON), 0, nullptr),
                     "Normalization3d::forward_propagate");
}

void Normalization3d::back_propagate(unique_ptr<LayerForwardPropagationCuda>& forward_propagation,
                                     unique_ptr<LayerBackPropagationCuda>& back_propagation) const
{
    Normalization3dForwardPropagationCuda* fp_cuda = static_cast<Normalization3dForwardPropagationCuda*>(forward_propagation.get());
    Normalization3dBackPropagationCuda* bp_cuda = static_cast<Normalization3dBackPropagationCuda*>(back_propagation.get());

    const int64_t rows = int64_t(fp_cuda->batch_size * sequence_length);
    const int64_t features = int64_t(get_embedding_dimension());

    // gradients of up to three consumers are summed on load: Layer::add_gradients (opennn/layer.cpp:447-457) is not needed
    const vector<TensorViewCuda>& deltas = back_propagation->output_gradients;
    if(deltas.size() > 3) add_gradients(deltas);

    // the stock propagation structures have no scratch view for this layer, so the entry point that needs none
    check_onn_status(onn_layernorm_bwd_static(deltas[0].data,
                                              deltas.size() > 1 && deltas.size() <= 3 ? deltas[1].data : nullptr,
                                              deltas.size() == 3 ? deltas[2].data : nullptr,
                                              forward_propagation->inputs[0].data,
                                              fp_cuda->means_device.data, fp_cuda->inv_variances_device.data,
                                              gammas_device.data,
                                              bp_cuda->input_gradients[0].data,
                                              bp_cuda->gamma_gradients.data, bp_cuda->beta_gradients.data,
                                              rows, features, 0, nullptr),
                     "Normalization3d::back_propagate");
}

}  // namespace opennn
