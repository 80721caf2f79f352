// Host mirror of NeuralNetwork, the Transformer builder and the propagation containers
// (opennn/neural_network.cpp, opennn/standard_networks.cpp:638-907).  The set() functions
// also work out the fusion plan described in opennn_b200.h.
#include <algorithm>
#include <cstring>

#include "opennn_b200.h"

namespace opennn_b200
{

// ---------------------------------------------------------------------------------------
// NeuralNetwork
// ---------------------------------------------------------------------------------------

void NeuralNetwork::add_layer(unique_ptr<Layer> layer, const vector<Index>& input_indices)
{
    // neural_network.cpp: with no indices given a layer reads the previous one
    const Index previous = get_layers_number() - 1;
    layer_input_indices.push_back(input_indices.empty() ? vector<Index>{previous} : input_indices);
    layers.push_back(std::move(layer));
}

vector<vector<Index>> NeuralNetwork::get_layer_output_indices() const
{
    vector<vector<Index>> outputs(layers.size());
    for(size_t consumer = 0; consumer < layers.size(); consumer++)
        for(const Index producer : layer_input_indices[consumer])
            if(producer >= 0) outputs[size_t(producer)].push_back(Index(consumer));
    return outputs;
}

Index NeuralNetwork::find_input_index(const vector<Index>& indices, Index layer_index) const
{
    for(size_t i = 0; i < indices.size(); i++)
        if(indices[i] == layer_index) return Index(i);
    throw std::runtime_error("find_input_index: layer is not an input of the consumer");
}

void NeuralNetwork::compile()
{
    // neural_network.cpp:66-94: one parameter arena, layer order, every view padded to 8 floats
    vector<vector<TensorViewCuda*>> views(layers.size());
    for(size_t i = 0; i < layers.size(); i++) views[i] = layers[i]->get_parameter_views_device();
    const Index total = get_size(views);
    parameters.assign(size_t(total), type(0));
    parameters_device.resize(total);
    link(parameters_device.data, views);
}

void NeuralNetwork::set_parameters_random(unsigned seed)
{
    Index offset = 0;
    for(size_t i = 0; i < layers.size(); i++)
    {
        layers[i]->set_parameters_random(parameters, offset, seed + unsigned(i) * 7919u);
        offset += layers[i]->get_parameters_number();
    }
    copy_parameters_device();
}

void NeuralNetwork::copy_parameters_device()
{
    check_cuda(cudaMemcpy(parameters_device.data, parameters.data(), parameters.size() * sizeof(type), cudaMemcpyHostToDevice),
               "copy_parameters_device");
    // a pageable-memory copy may return before its DMA has landed; later work runs on other streams
    check_cuda(cudaDeviceSynchronize(), "copy_parameters_device");
}

void NeuralNetwork::copy_parameters_host()
{
    check_cuda(cudaMemcpy(parameters.data(), parameters_device.data, parameters.size() * sizeof(type), cudaMemcpyDeviceToHost),
               "copy_parameters_host");
}

vector<char> NeuralNetwork::layers_depending_on_input(Index external) const
{
    vector<char> depends(layers.size(), 0);
    for(size_t i = 0; i < layers.size(); i++)                  // layers are stored in topological order
        for(const Index source : layer_input_indices[i])
            if(source == -external || (source >= 0 && depends[size_t(source)])) depends[i] = 1;
    return depends;
}

void NeuralNetwork::forward_propagate(const vector<TensorViewCuda>& input_views, ForwardPropagationCuda& forward_propagation, bool is_training,
                                      const vector<char>* run_layer)
{
    // neural_network.cpp:1889-1943: external input -k is input_views[k-1]
    for(size_t i = 0; i < layers.size(); i++)
    {
        if(run_layer && !(*run_layer)[i]) continue;
        unique_ptr<LayerForwardPropagationCuda>& state = forward_propagation.layers[i];
        for(size_t port = 0; port < layer_input_indices[i].size(); port++)
        {
            const Index source = layer_input_indices[i][port];
            if(source < 0)
            {
                const size_t external = size_t(-source - 1);
                if(external >= input_views.size()) throw std::runtime_error("forward_propagate: missing external input");
                state->inputs[port] = input_views[external];
            }
        }
        if(before_layer_hook) before_layer_hook(before_layer_context, Index(i));
        layers[i]->forward_propagate(state, is_training);
    }
}


// ---------------------------------------------------------------------------------------
// Transformer (standard_networks.cpp:638-907) and the decoder-only stack
// ---------------------------------------------------------------------------------------

static string suffix_of(Index i) { return "_" + std::to_string(i + 1); }

Transformer::Transformer(Index input_sequence_length, Index decoder_sequence_length, Index input_vocabulary_size,
                         Index output_vocabulary_size, Index embedding_dimension, Index heads_number,
                         Index feed_forward_dimension, Index layers_number)
{
    if(embedding_dimension % heads_number != 0)
        throw std::runtime_error("Transformer Error: embedding_dimension must be divisible by heads_number.");

    const Shape input_shape = {input_sequence_length, embedding_dimension};
    const Shape decoder_shape = {decoder_sequence_length, embedding_dimension};

    auto decoder_embedding = std::make_unique<Embedding>(Shape{output_vocabulary_size, decoder_sequence_length}, embedding_dimension, "decoder_embedding");
    decoder_embedding->set_scale_embedding(true);
    decoder_embedding->set_add_positional_encoding(true);
    add_layer(std::move(decoder_embedding), {-1});
    Index current_decoder = get_layers_number() - 1;

    auto encoder_embedding = std::make_unique<Embedding>(Shape{input_vocabulary_size, input_sequence_length}, embedding_dimension, "encoder_embedding");
    encoder_embedding->set_scale_embedding(true);
    encoder_embedding->set_add_positional_encoding(true);
    add_layer(std::move(encoder_embedding), {-2});
    Index current_encoder = get_layers_number() - 1;

    for(Index i = 0; i < layers_number; i++)
    {
        const string suffix = suffix_of(i);
        add_layer(std::make_unique<MultiHeadAttention>(input_shape, heads_number, "encoder_self_attention" + suffix), {current_encoder});
        const Index attention = get_layers_number() - 1;
        add_layer(std::make_unique<Addition3d>(input_shape, "encoder_self_attention_addition" + suffix), {current_encoder, attention});
        add_layer(std::make_unique<Normalization3d>(input_shape, "encoder_self_attention_normalization" + suffix));
        const Index norm_1 = get_layers_number() - 1;
        add_layer(std::make_unique<Dense3d>(input_sequence_length, embedding_dimension, feed_forward_dimension, "RectifiedLinear", "encoder_internal_dense" + suffix));
        add_layer(std::make_unique<Dense3d>(input_sequence_length, feed_forward_dimension, embedding_dimension, "Linear", "encoder_external_dense" + suffix));
        const Index dense = get_layers_number() - 1;
        add_layer(std::make_unique<Addition3d>(input_shape, "encoder_dense_addition" + suffix), {norm_1, dense});
        add_layer(std::make_unique<Normalization3d>(input_shape, "encoder_dense_normalization" + suffix));
        current_encoder = get_layers_number() - 1;
    }
    const Index encoder_output = current_encoder;

    for(Index i = 0; i < layers_number; i++)
    {
        const string suffix = suffix_of(i);
        auto self_attention = std::make_unique<MultiHeadAttention>(decoder_shape, heads_number, "decoder_self_attention" + suffix);
        self_attention->set(decoder_sequence_length, decoder_sequence_length, embedding_dimension, heads_number, true, "decoder_self_attention" + suffix);
        add_layer(std::move(self_attention), {current_decoder});
        const Index attention = get_layers_number() - 1;
        add_layer(std::make_unique<Addition3d>(decoder_shape, "decoder_self_attention_addition" + suffix), {current_decoder, attention});
        add_layer(std::make_unique<Normalization3d>(decoder_shape, "decoder_self_attention_normalization" + suffix));
        const Index norm_1 = get_layers_number() - 1;
        add_layer(std::make_unique<MultiHeadAttention>(decoder_shape, input_shape, heads_number, "cross_attention" + suffix), {norm_1, encoder_output});
        const Index cross = get_layers_number() - 1;
        add_layer(std::make_unique<Addition3d>(decoder_shape, "cross_attention_addition" + suffix), {norm_1, cross});
        add_layer(std::make_unique<Normalization3d>(decoder_shape, "cross_attention_normalization" + suffix));
        const Index norm_2 = get_layers_number() - 1;
        add_layer(std::make_unique<Dense3d>(decoder_sequence_length, embedding_dimension, feed_forward_dimension, "RectifiedLinear", "decoder_internal_dense" + suffix));
        add_layer(std::make_unique<Dense3d>(decoder_sequence_length, feed_forward_dimension, embedding_dimension, "Linear", "decoder_external_dense" + suffix));
        const Index dense = get_layers_number() - 1;
        add_layer(std::make_unique<Addition3d>(decoder_shape, "decoder_dense_addition" + suffix), {norm_2, dense});
        add_layer(std::make_unique<Normalization3d>(decoder_shape, "decoder_dense_normalization" + suffix));
        current_decoder = get_layers_number() - 1;
    }

    add_layer(std::make_unique<Dense3d>(decoder_sequence_length, embedding_dimension, output_vocabulary_size, "Softmax", "output_projection"));
    compile();
    set_parameters_random();
}

TextClassificationNetwork::TextClassificationNetwork(Index vocabulary_size, Index sequence_length, Index embedding_dimension, Index heads_number,
                                                     const vector<Index>& complexity_dimensions, Index classes)
{
    if(classes < 1) throw std::runtime_error("TextClassificationNetwork: at least one output.");
    auto embedding = std::make_unique<Embedding>(Shape{vocabulary_size, sequence_length}, embedding_dimension, "embedding_layer");
    embedding->set_scale_embedding(true);
    embedding->set_add_positional_encoding(true);
    add_layer(std::move(embedding), {-1});
    add_layer(std::make_unique<MultiHeadAttention>(Shape{sequence_length, embedding_dimension}, heads_number, "multihead_attention_layer"), {0});
    add_layer(std::make_unique<Pooling3d>(Shape{sequence_length, embedding_dimension}, Pooling3d::PoolingMethod::MaxPooling), {1});
    Index width = embedding_dimension;
    for(size_t i = 0; i < complexity_dimensions.size(); i++)
    {
        add_layer(Dense3d::make_rank2(width, complexity_dimensions[i], "RectifiedLinear", "dense2d_layer_" + std::to_string(i + 1)),
                  {get_layers_number() - 1});
        width = complexity_dimensions[i];
    }
    add_layer(Dense3d::make_rank2(width, classes, classes > 1 ? "Softmax" : "Sigmoid", "classification_layer"), {get_layers_number() - 1});
    compile();
    set_parameters_random();
}

unique_ptr<NeuralNetwork> make_decoder_only_network(Index sequence_length, Index vocabulary_size, Index embedding_dimension,
                                                    Index heads_number, Index feed_forward_dimension, Index layers_number)
{
    auto network = std::make_unique<NeuralNetwork>();
    const Shape shape = {sequence_length, embedding_dimension};
    auto embedding = std::make_unique<Embedding>(Shape{vocabulary_size, sequence_length}, embedding_dimension, "decoder_embedding");
    embedding->set_scale_embedding(true);
    embedding->set_add_positional_encoding(true);
    network->add_layer(std::move(embedding), {-1});
    Index current = network->get_layers_number() - 1;
    for(Index i = 0; i < layers_number; i++)
    {
        const string suffix = suffix_of(i);
        auto attention_layer = std::make_unique<MultiHeadAttention>(shape, heads_number, "decoder_self_attention" + suffix);
        attention_layer->set(sequence_length, sequence_length, embedding_dimension, heads_number, true, "decoder_self_attention" + suffix);
        network->add_layer(std::move(attention_layer), {current});
        const Index attention = network->get_layers_number() - 1;
        network->add_layer(std::make_unique<Addition3d>(shape, "decoder_self_attention_addition" + suffix), {current, attention});
        network->add_layer(std::make_unique<Normalization3d>(shape, "decoder_self_attention_normalization" + suffix));
        const Index norm_1 = network->get_layers_number() - 1;
        network->add_layer(std::make_unique<Dense3d>(sequence_length, embedding_dimension, feed_forward_dimension, "RectifiedLinear", "decoder_internal_dense" + suffix));
        network->add_layer(std::make_unique<Dense3d>(sequence_length, feed_forward_dimension, embedding_dimension, "Linear", "decoder_external_dense" + suffix));
        const Index dense = network->get_layers_number() - 1;
        network->add_layer(std::make_unique<Addition3d>(shape, "decoder_dense_addition" + suffix), {norm_1, dense});
        network->add_layer(std::make_unique<Normalization3d>(shape, "decoder_dense_normalization" + suffix));
        current = network->get_layers_number() - 1;
    }
    network->add_layer(std::make_unique<Dense3d>(sequence_length, embedding_dimension, vocabulary_size, "Softmax", "output_projection"));
    network->compile();
    network->set_parameters_random();
    return network;
}


// ---------------------------------------------------------------------------------------
// ForwardPropagationCuda (neural_network.cpp:1983-2028)
// ---------------------------------------------------------------------------------------

ForwardPropagationCuda::ForwardPropagationCuda(Index new_samples_number, NeuralNetwork* new_neural_network)
{
    if(new_neural_network) set(new_samples_number, new_neural_network);
}

void ForwardPropagationCuda::set(Index new_samples_number, NeuralNetwork* new_neural_network)
{
    samples_number = new_samples_number;
    neural_network = new_neural_network;
    if(!neural_network) throw std::runtime_error("There is no neural network.");

    const vector<unique_ptr<Layer>>& network_layers = neural_network->get_layers();
    const vector<vector<Index>>& input_indices = neural_network->get_layer_input_indices();
    const vector<vector<Index>> output_indices = neural_network->get_layer_output_indices();
    const size_t layers_number = network_layers.size();

    layers.resize(layers_number);
    for(size_t i = 0; i < layers_number; i++)
    {
        layers[i] = network_layers[i]->create_forward_propagation();
        layers[i]->set(samples_number, network_layers[i].get());
    }

    // plan: which producers must also emit key-padding flags (their output is the SOURCE of an attention layer)
    for(size_t i = 0; i < layers_number; i++)
    {
        if(network_layers[i]->get_name() != "MultiHeadAttention") continue;
        const Index source = input_indices[i].size() > 1 ? input_indices[i][1] : input_indices[i][0];
        if(source < 0) continue;
        const string& producer = network_layers[size_t(source)]->get_name();
        if(producer == "Embedding" || producer == "Normalization3d") layers[size_t(source)]->wants_row_flags = true;
    }

    // plan: a Dense "RectifiedLinear" read by one Dense layer only also writes its ReLU mask as bits; that consumer's
    // input-gradient GEMM applies the mask (see NeuralNetworkBackPropagationCuda::set, which makes the same test)
    for(size_t i = 0; i < layers_number; i++)
    {
        const Dense3d* dense = dynamic_cast<const Dense3d*>(network_layers[i].get());
        if(!dense || dense->get_activation_function() != "RectifiedLinear" || output_indices[i].size() != 1) continue;
        const size_t consumer = size_t(output_indices[i][0]);
        if(network_layers[consumer]->get_name() != "Dense3d" || input_indices[consumer].size() != 1) continue;
        static_cast<Dense3dForwardPropagationCuda*>(layers[i].get())->wants_relu_bits = true;
    }

    vector<vector<TensorViewCuda*>> views(layers_number);
    for(size_t i = 0; i < layers_number; i++) views[i] = layers[i]->get_workspace_views();
    workspace.resize(get_size(views));
    link(workspace.data, views);

    // wiring: a consumer's inputs are views of its producers' outputs (neural_network.cpp:2016-2027)
    for(size_t i = 0; i < layers_number; i++)
    {
        layers[i]->inputs.clear();
        for(const Index source : input_indices[i])
            layers[i]->inputs.push_back(source >= 0 ? layers[size_t(source)]->outputs : TensorViewCuda());
    }

    for(size_t i = 0; i < layers_number; i++)
    {
        const string& name = network_layers[i]->get_name();

        if(name == "MultiHeadAttention")
        {
            const Index source = input_indices[i].size() > 1 ? input_indices[i][1] : input_indices[i][0];
            if(source >= 0 && layers[size_t(source)]->wants_row_flags)
                static_cast<MultiHeadAttentionForwardPropagationCuda*>(layers[i].get())->source_row_is_zero =
                    reinterpret_cast<const uint8_t*>(layers[size_t(source)]->outputs_row_is_zero.data);
        }

        // plan: Addition<3> read only by a Normalization3d is computed inside that layer's kernel
        if(name == "Addition3d" && output_indices[i].size() == 1 &&
           network_layers[size_t(output_indices[i][0])]->get_name() == "Normalization3d" &&
           input_indices[i].size() == 2 && input_indices[i][0] >= 0 && input_indices[i][1] >= 0)
        {
            layers[i]->fused_into_consumer = true;
            auto* norm = static_cast<Normalization3dForwardPropagationCuda*>(layers[size_t(output_indices[i][0])].get());
            norm->addend_a = layers[i]->inputs[0].data;
            norm->addend_b = layers[i]->inputs[1].data;
            norm->sum_output = layers[i]->outputs.data;
        }
    }
}


// ---------------------------------------------------------------------------------------
// NeuralNetworkBackPropagationCuda (neural_network.cpp:2096-2161)
// ---------------------------------------------------------------------------------------

void NeuralNetworkBackPropagationCuda::set(Index new_batch_size, NeuralNetwork* new_neural_network, ForwardPropagationCuda* forward_propagation)
{
    batch_size = new_batch_size;
    neural_network = new_neural_network;
    if(!neural_network) return;

    const vector<unique_ptr<Layer>>& network_layers = neural_network->get_layers();
    const vector<vector<Index>>& input_indices = neural_network->get_layer_input_indices();
    const vector<vector<Index>> output_indices = neural_network->get_layer_output_indices();
    const size_t layers_number = network_layers.size();

    layers.resize(layers_number);
    for(size_t i = 0; i < layers_number; i++)
    {
        layers[i] = network_layers[i]->create_back_propagation();
        layers[i]->set(batch_size, network_layers[i].get());
    }

    // gradients: one arena with the parameters' layout (neural_network.cpp:2117-2124)
    vector<vector<TensorViewCuda*>> gradient_views(layers_number);
    for(size_t i = 0; i < layers_number; i++) gradient_views[i] = layers[i]->get_gradient_views();
    gradients.resize(get_size(gradient_views));
    link(gradients.data, gradient_views);

    // plan 1: Addition<3> fused into the following Normalization3d -- its two input gradients are the
    // consumer's input gradient (addition_layer.h:148-168 copies the same tensor to both)
    for(size_t i = 0; i < layers_number; i++)
        if(forward_propagation && forward_propagation->layers[i]->fused_into_consumer)
        {
            layers[i]->fused_into_consumer = true;
            layers[i]->owns_input_gradient.assign(2, false);
        }

    // plan 2: every cross-attention layer that reads the same source shares one source-gradient buffer;
    // the one that runs first in the reverse walk (highest index) overwrites, the others accumulate
    vector<Index> source_gradient_owner(layers_number, -1);
    for(size_t producer = 0; producer < layers_number; producer++)
    {
        Index owner = -1;
        for(const Index consumer : output_indices[producer])
        {
            const bool cross_source = network_layers[size_t(consumer)]->get_name() == "MultiHeadAttention" &&
                                      input_indices[size_t(consumer)].size() > 1 && input_indices[size_t(consumer)][1] == Index(producer);
            if(!cross_source) continue;
            if(owner < 0 || consumer > owner) owner = consumer;
        }
        for(const Index consumer : output_indices[producer])
        {
            const bool cross_source = network_layers[size_t(consumer)]->get_name() == "MultiHeadAttention" &&
                                      input_indices[size_t(consumer)].size() > 1 && input_indices[size_t(consumer)][1] == Index(producer);
            if(!cross_source || consumer == owner) continue;
            layers[size_t(consumer)]->owns_input_gradient[1] = false;
            layers[size_t(consumer)]->accumulate_input_gradient[1] = true;
            source_gradient_owner[size_t(consumer)] = owner;
        }
    }

    // plan 3: Dense "Linear" fed by a Dense "RectifiedLinear" that nobody else reads
    vector<std::pair<size_t, size_t>> fused_relu_pairs;
    for(size_t i = 0; i < layers_number; i++)
    {
        if(network_layers[i]->get_name() != "Dense3d" || input_indices[i].size() != 1 || input_indices[i][0] < 0) continue;
        const size_t producer = size_t(input_indices[i][0]);
        const Dense3d* producer_dense = dynamic_cast<const Dense3d*>(network_layers[producer].get());
        if(!producer_dense || producer_dense->get_activation_function() != "RectifiedLinear" || output_indices[producer].size() != 1) continue;
        if(!forward_propagation) continue;
        static_cast<Dense3dBackPropagationCuda*>(layers[i].get())->input_relu_mask = forward_propagation->layers[producer]->outputs.data;
        const auto* producer_forward = static_cast<const Dense3dForwardPropagationCuda*>(forward_propagation->layers[producer].get());
        if(producer_forward->wants_relu_bits)
            static_cast<Dense3dBackPropagationCuda*>(layers[i].get())->input_relu_bits = reinterpret_cast<const uint32_t*>(producer_forward->relu_bits.data);
        static_cast<Dense3dBackPropagationCuda*>(layers[producer].get())->delta_is_ready = true;
        fused_relu_pairs.push_back({i, producer});
    }

    for(const auto& pair : fused_relu_pairs)
    {
        auto* consumer = static_cast<Dense3dBackPropagationCuda*>(layers[pair.first].get());
        auto* producer = static_cast<Dense3dBackPropagationCuda*>(layers[pair.second].get());
        consumer->input_bias_gradients = producer->bias_gradients.data;     // the gradient arena is linked by now
        producer->bias_gradient_is_ready = true;
    }

    // plan 4: Normalization3d over a fused Addition<3> one of whose addends comes from a Dense "Linear" or a
    // MultiHeadAttention layer that nobody else reads: that layer's output gradient IS the normalisation's input
    // gradient, so its (projection) bias gradient is the column sum of that tensor, which the normalisation kernel takes
    for(size_t i = 0; i < layers_number; i++)
    {
        if(network_layers[i]->get_name() != "Normalization3d" || input_indices[i].size() != 1 || input_indices[i][0] < 0) continue;
        const size_t addition = size_t(input_indices[i][0]);
        if(!layers[addition]->fused_into_consumer) continue;
        for(const Index addend : input_indices[addition])
        {
            if(addend < 0 || output_indices[size_t(addend)].size() != 1) continue;
            auto* norm = static_cast<Normalization3dBackPropagationCuda*>(layers[i].get());
            if(norm->input_bias_gradients) break;
            if(auto* dense = dynamic_cast<Dense3dBackPropagationCuda*>(layers[size_t(addend)].get()))
            {
                const Dense3d* dense_layer = static_cast<const Dense3d*>(network_layers[size_t(addend)].get());
                if(dense_layer->get_activation_function() != "Linear" || dense->bias_gradient_is_ready) continue;
                norm->input_bias_gradients = dense->bias_gradients.data;
                dense->bias_gradient_is_ready = true;
            }
            else if(auto* attention = dynamic_cast<MultiHeadAttentionBackPropagationCuda*>(layers[size_t(addend)].get()))
            {
                norm->input_bias_gradients = attention->projection_bias_gradients.data;
                attention->projection_bias_gradient_is_ready = true;
            }
        }
    }

    // workspace: the input gradients each layer owns, plus per-layer scratch
    vector<vector<TensorViewCuda*>> workspace_views(layers_number);
    for(size_t i = 0; i < layers_number; i++) workspace_views[i] = layers[i]->get_workspace_views();
    workspace.resize(get_size(workspace_views));
    link(workspace.data, workspace_views);

    // aliases
    for(size_t i = 0; i < layers_number; i++)
        if(source_gradient_owner[i] >= 0)
            layers[i]->input_gradients[1].data = layers[size_t(source_gradient_owner[i])]->input_gradients[1].data;

    Index attention_scratch_floats = 0;
    for(size_t i = 0; i < layers_number; i++)
        if(auto* attention = dynamic_cast<MultiHeadAttentionBackPropagationCuda*>(layers[i].get()))
            attention_scratch_floats = std::max(attention_scratch_floats, attention->scratch_floats);
    attention_scratch.resize(attention_scratch_floats);
    for(size_t i = 0; i < layers_number; i++)
        if(auto* attention = dynamic_cast<MultiHeadAttentionBackPropagationCuda*>(layers[i].get()))
            attention->scratch = TensorViewCuda(attention_scratch.data, {attention_scratch_floats});

    // output gradients of each producer = input gradients of its consumers (neural_network.cpp:2140-2160);
    // consumers that share a buffer contribute it once; a fused Addition<3> passes its consumer's gradient through
    for(Index i = Index(layers_number) - 1; i >= 0; i--)
    {
        LayerBackPropagationCuda& state = *layers[size_t(i)];
        state.output_gradients.clear();
        if(i == Index(layers_number) - 1) { state.output_gradients.push_back(TensorViewCuda()); continue; }
        for(const Index consumer : output_indices[size_t(i)])
        {
            const Index port = neural_network->find_input_index(input_indices[size_t(consumer)], i);
            const TensorViewCuda& view = layers[size_t(consumer)]->input_gradients[size_t(port)];
            bool seen = false;
            for(const TensorViewCuda& existing : state.output_gradients) seen = seen || existing.data == view.data;
            if(!seen) state.output_gradients.push_back(view);
        }
        if(state.fused_into_consumer)
        {
            // the Normalization3d that computes this addition writes the gradient of the sum; both addends receive it
            state.input_gradients[0].data = state.output_gradients[0].data;
            state.input_gradients[1].data = state.output_gradients[0].data;
        }
    }
}

}  // namespace opennn_b200
