// Host mirror of CrossEntropyError3d / Loss::back_propagate (opennn/cross_entropy_error_3d.cpp,
// opennn/loss.cpp:1249-1289) and AdaptiveMomentEstimation::update_parameters
// (opennn/adaptive_moment_estimation.cpp:855-883 with the CPU path's clip, :462-466).
#include <cmath>

#include "opennn_b200.h"

namespace opennn_b200
{

static void* stream() { return Device::instance().get_compute_stream(); }

constexpr Index kStatisticSlots = 64;     // micro-batches whose loss statistics can be held before one read

vector<TensorViewCuda> BatchCuda::get_inputs_device() const
{
    // dataset.cpp:4331-4339: {decoder, input} when there is a decoder input, else {input}
    vector<TensorViewCuda> views;
    if(decoder.data) views.push_back(decoder);
    if(input.data) views.push_back(input);
    return views;
}

BackPropagationCuda::BackPropagationCuda(Index new_samples_number, CrossEntropyError3d* new_loss, ForwardPropagationCuda* forward_propagation)
{
    if(new_loss) set(new_samples_number, new_loss, forward_propagation);
}

BackPropagationCuda::~BackPropagationCuda()
{
    if(pinned_statistics) cudaFreeHost(pinned_statistics);
}

void BackPropagationCuda::set(Index new_samples_number, CrossEntropyError3d* new_loss, ForwardPropagationCuda* forward_propagation)
{
    samples_number = new_samples_number;
    loss = new_loss;
    NeuralNetwork* network = loss->get_neural_network();
    neural_network.set(samples_number, network, forward_propagation);

    // the output layer's buffer doubles as the output-gradient buffer: the fused loss kernel
    // turns logits into gradients in place (loss.cpp:1375-1435 allocates a second [B,S,V] tensor)
    if(forward_propagation)
    {
        output_gradients = forward_propagation->layers.back()->outputs;
        if(auto* dense = dynamic_cast<Dense3dForwardPropagationCuda*>(forward_propagation->layers.back().get()))
            if(static_cast<const Dense3d*>(dense->layer)->get_activation_function() == "Softmax")
                dense->defer_softmax = true;
    }

    const Shape output_shape = network->get_output_shape();
    statistics.resize(4 * kStatisticSlots);
    active_count.resize(8);
    row_scratch.resize(2 * samples_number * output_shape[0]);
    check_cuda(cudaMallocHost(reinterpret_cast<void**>(&pinned_statistics), 4 * kStatisticSlots * sizeof(type)), "pinned statistics");
}

void CrossEntropyError3d::set_regularization_method(const string& method)
{
    if(method != "None")
        throw std::runtime_error("CrossEntropyError3d: only regularization \"None\" is implemented on this path (OpenNN's default is L2).");
    regularization_method = method;
}

void CrossEntropyError3d::calculate_active_tokens(const BatchCuda& batch, BackPropagationCuda& back_propagation) const
{
    const Index vocabulary_size = neural_network->get_output_shape().back();
    check_onn(onn_ce3d_count_active(batch.target.data, batch.target.size(), vocabulary_size, back_propagation.active_count.data, stream()),
              "CrossEntropyError3d::calculate_active_tokens");
}


void CrossEntropyError3d::calculate_error_and_output_gradients(const BatchCuda& batch, ForwardPropagationCuda& forward_propagation,
                                                               BackPropagationCuda& back_propagation, bool accumulate_statistics) const
{
    const TensorViewCuda outputs = forward_propagation.get_last_trainable_layer_outputs_device();
    const Index vocabulary_size = outputs.shape.back();
    const Index rows = outputs.size() / vocabulary_size;
    if(vocabulary_size == 1)
        throw std::runtime_error("CrossEntropyError3d: the binary (one output) variant is not implemented on this path.");

    bool deferred = false;
    if(auto* dense = dynamic_cast<Dense3dForwardPropagationCuda*>(forward_propagation.layers.back().get())) deferred = dense->defer_softmax;

    if(!accumulate_statistics) back_propagation.statistics_slot = 0;
    if(back_propagation.statistics_slot >= kStatisticSlots) throw std::runtime_error("CrossEntropyError3d: too many micro-batches before read_error");
    type* statistics = back_propagation.statistics.data + 4 * back_propagation.statistics_slot++;

    check_onn(onn_ce3d_fwd_bwd(outputs.data, batch.target.data, back_propagation.active_count.data, nullptr, statistics,
                               back_propagation.row_scratch.data, rows, vocabulary_size, deferred ? 0 : 1, 0, stream()),
              "CrossEntropyError3d::calculate_error_and_output_gradients");
}

void CrossEntropyError3d::calculate_layers_error_gradient(ForwardPropagationCuda& forward_propagation, BackPropagationCuda& back_propagation) const
{
    // loss.cpp:1271-1289
    const vector<unique_ptr<Layer>>& layers = neural_network->get_layers();
    const Index last = neural_network->get_last_trainable_layer_index();
    const Index first = neural_network->get_first_trainable_layer_index();
    back_propagation.neural_network.layers[size_t(last)]->output_gradients[0] = back_propagation.get_output_gradients_device();
    for(Index i = last; i >= first; i--)
    {
        layers[size_t(i)]->back_propagate(forward_propagation.layers[size_t(i)], back_propagation.neural_network.layers[size_t(i)]);
        if(gradient_ready_hook) gradient_ready_hook(gradient_ready_context, i);
    }
}

void CrossEntropyError3d::back_propagate(const BatchCuda& batch, ForwardPropagationCuda& forward_propagation,
                                         BackPropagationCuda& back_propagation, bool accumulate_statistics) const
{
    // loss.cpp:1249-1268 without the two blocking device-to-host copies of calculate_error
    if(batch.is_empty()) return;
    calculate_error_and_output_gradients(batch, forward_propagation, back_propagation, accumulate_statistics);
    calculate_layers_error_gradient(forward_propagation, back_propagation);
}

void CrossEntropyError3d::read_error(BackPropagationCuda& back_propagation, type global_active_tokens) const
{
    const Index slots = back_propagation.statistics_slot;
    cudaStream_t s = Device::instance().get_compute_stream();
    check_cuda(cudaMemcpyAsync(back_propagation.pinned_statistics, back_propagation.statistics.data, size_t(4 * slots) * sizeof(type),
                               cudaMemcpyDeviceToHost, s), "read_error");
    check_cuda(cudaStreamSynchronize(s), "read_error sync");
    double loss_sum = 0, correct = 0, active = 0;
    for(Index k = 0; k < slots; k++)
    {
        loss_sum += back_propagation.pinned_statistics[4 * k];
        correct += back_propagation.pinned_statistics[4 * k + 1];
        active += back_propagation.pinned_statistics[4 * k + 2];
    }
    if(global_active_tokens > 0) active = global_active_tokens;
    back_propagation.error = active > 0 ? type(loss_sum / active) : type(0);
    back_propagation.accuracy = active > 0 ? type(correct / active) : type(0);
    back_propagation.loss_value = back_propagation.error;
    if(std::isnan(back_propagation.error)) throw std::runtime_error("Error is NAN.");      // cross_entropy_error_3d.cpp:452-453
}


// ---------------------------------------------------------------------------------------
// CrossEntropyError2d
// ---------------------------------------------------------------------------------------

void CrossEntropyError2d::back_propagate(const TensorViewCuda& targets, ForwardPropagationCuda& forward_propagation,
                                         NeuralNetworkBackPropagationCuda& back_propagation, type* statistics, type* row_scratch) const
{
    const vector<unique_ptr<Layer>>& layers = neural_network->get_layers();
    const Index last = neural_network->get_last_trainable_layer_index();
    const Index first = neural_network->get_first_trainable_layer_index();
    const TensorViewCuda outputs = forward_propagation.layers[size_t(last)]->outputs;
    const Index classes = outputs.shape.back();
    const Index samples = outputs.size() / classes;
    if(targets.size() != samples * classes) throw std::runtime_error("CrossEntropyError2d: targets must be [samples, classes]");
    if(classes == 1)
    {
        // binary form: the output buffer doubles as the gradient buffer, so the kernel leaves the Sigmoid layer's delta
        auto* dense_back = dynamic_cast<Dense3dBackPropagationCuda*>(back_propagation.layers[size_t(last)].get());
        const Dense3d* dense = dynamic_cast<const Dense3d*>(layers[size_t(last)].get());
        if(!dense_back || !dense || dense->get_activation_code() != ONN_ACT_SIGMOID)
            throw std::runtime_error("CrossEntropyError2d: one output needs a Dense \"Sigmoid\" output layer on this path.");
        dense_back->delta_is_ready = true;
        check_onn(onn_ce2d_binary_fwd_bwd(outputs.data, targets.data, statistics, row_scratch, samples, 1, stream()),
                  "CrossEntropyError2d::back_propagate");
    }
    else
        check_onn(onn_ce2d_fwd_bwd(outputs.data, targets.data, statistics, row_scratch, samples, classes, stream()),
                  "CrossEntropyError2d::back_propagate");
    back_propagation.layers[size_t(last)]->output_gradients[0] = outputs;
    for(Index i = last; i >= first; i--)
        layers[size_t(i)]->back_propagate(forward_propagation.layers[size_t(i)], back_propagation.layers[size_t(i)]);
}


// ---------------------------------------------------------------------------------------
// AdaptiveMomentEstimation
// ---------------------------------------------------------------------------------------

ADAMOptimizationDataCuda::ADAMOptimizationDataCuda(AdaptiveMomentEstimation* optimizer)
{
    if(optimizer) set(optimizer);
}

void ADAMOptimizationDataCuda::set(AdaptiveMomentEstimation* optimizer)
{
    adaptive_moment_estimation = optimizer;
    set(optimizer->get_loss()->get_neural_network()->get_parameters_number());
}

void ADAMOptimizationDataCuda::set(Index parameters_number)
{
    gradient_exponential_decay.resize(parameters_number);
    square_gradient_exponential_decay.resize(parameters_number);
    square_norm.resize(8);
    norm_workspace.resize(Index(onn_grad_sqnorm_workspace_floats(parameters_number)));
    iteration = 1;
}

void AdaptiveMomentEstimation::update_parameters(BackPropagationCuda& back_propagation, ADAMOptimizationDataCuda& optimization_data,
                                                 type gradient_scale) const
{
    update_parameters(loss->get_neural_network(), back_propagation.neural_network.gradients, optimization_data, gradient_scale);
}

void AdaptiveMomentEstimation::update_parameters(NeuralNetwork* network, TensorCuda& gradients, ADAMOptimizationDataCuda& optimization_data,
                                                 type gradient_scale) const
{
    type bias_correction_1, bias_correction_2;
    advance(optimization_data, bias_correction_1, bias_correction_2);

    const Index n = network->get_parameters_number();
    check_onn(onn_grad_sqnorm(gradients.data, n, optimization_data.square_norm.data, optimization_data.norm_workspace.data, stream()),
              "AdaptiveMomentEstimation: gradient norm");
    check_onn(onn_adam_guarded(network->get_parameters_device().data, optimization_data.gradient_exponential_decay.data,
                               optimization_data.square_gradient_exponential_decay.data, gradients.data, n,
                               learning_rate, beta_1, beta_2, EPSILON, bias_correction_1, bias_correction_2,
                               gradient_clip_norm, optimization_data.square_norm.data, gradient_scale, 1, skip_if_nonzero, stream()),
              "AdaptiveMomentEstimation::update_parameters");
}

void AdaptiveMomentEstimation::advance(ADAMOptimizationDataCuda& optimization_data, type& bias_correction_1, type& bias_correction_2) const
{
    optimization_data.iteration++;
    const type iteration = type(optimization_data.iteration);
    bias_correction_1 = type(1) - std::pow(beta_1, iteration);
    bias_correction_2 = type(1) - std::pow(beta_2, iteration);
}

}  // namespace opennn_b200
