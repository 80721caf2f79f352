// Incremental decoding for the Transformer of this mirror: one target position per step, keys and values cached.
// See the class comment in opennn_b200.h.  Every device computation goes through the C ABI of onn_b200.h.
#include <algorithm>
#include <memory>
#include <stdexcept>

#include "opennn_b200.h"

namespace opennn_b200
{

static void* stream() { return Device::instance().get_compute_stream(); }

IncrementalDecoder::IncrementalDecoder(NeuralNetwork* new_network, ForwardPropagationCuda* new_forward_propagation, Index new_batch_size)
    : network(new_network), forward_propagation(new_forward_propagation), batch_size(new_batch_size)
{
    const vector<unique_ptr<Layer>>& layers = network->get_layers();
    decoder_side = network->layers_depending_on_input(1);
    outputs.resize(layers.size());
    caches.resize(layers.size());
    Index widest = 0;
    for(size_t i = 0; i < layers.size(); i++)
    {
        if(!decoder_side[i]) continue;
        const Shape shape = layers[i]->get_output_shape();          // {sequence, features}
        outputs[i] = std::make_unique<TensorCuda>();
        outputs[i]->resize(batch_size * shape.back());
        widest = std::max(widest, shape.back());
        if(const MultiHeadAttention* attention = dynamic_cast<const MultiHeadAttention*>(layers[i].get()))
        {
            caches[i] = std::make_unique<AttentionCache>();
            AttentionCache& cache = *caches[i];
            cache.capacity = attention->get_source_sequence_length();
            cache.keys.resize(batch_size * cache.capacity * attention->get_embedding_dimension());
            cache.values.resize(batch_size * cache.capacity * attention->get_embedding_dimension());
            cache.key_is_pad.resize((batch_size * cache.capacity + 3) / 4);       // bytes, held in a float buffer
        }
    }
    query.resize(batch_size * widest);
    context.resize(batch_size * widest);
    step_ids.resize(batch_size);
}

void IncrementalDecoder::start()
{
    const vector<unique_ptr<Layer>>& layers = network->get_layers();
    const vector<vector<Index>>& input_indices = network->get_layer_input_indices();
    for(size_t i = 0; i < layers.size(); i++)
    {
        const MultiHeadAttention* attention = dynamic_cast<const MultiHeadAttention*>(layers[i].get());
        if(!attention || !decoder_side[i] || !attention->is_cross_attention()) continue;
        // keys and values of the encoder output, once: K = Xs Wk + bk, V = Xs Wv + bv, padding flags of Xs
        const Index source = input_indices[i][1];
        if(source < 0 || decoder_side[size_t(source)]) throw std::runtime_error("IncrementalDecoder: a cross-attention source must be an encoder-side layer");
        const type* encoder_output = forward_propagation->layers[size_t(source)]->outputs.data;
        const Index rows = batch_size * attention->get_source_sequence_length(), E = attention->get_embedding_dimension();
        AttentionCache& cache = *caches[i];
        check_onn(onn_dense_fwd(encoder_output, attention->key_weights_device.data, attention->key_biases_device.data, cache.keys.data, nullptr,
                                rows, E, E, ONN_ACT_LINEAR, 0, stream()), "IncrementalDecoder: cross keys");
        check_onn(onn_dense_fwd(encoder_output, attention->value_weights_device.data, attention->value_biases_device.data, cache.values.data, nullptr,
                                rows, E, E, ONN_ACT_LINEAR, 0, stream()), "IncrementalDecoder: cross values");
        check_onn(onn_rows_are_zero(encoder_output, reinterpret_cast<uint8_t*>(cache.key_is_pad.data), rows, E, stream()), "IncrementalDecoder: cross padding");
    }
}

const type* IncrementalDecoder::step(const type* ids, Index ids_stride, Index position, bool output_logits)
{
    const vector<unique_ptr<Layer>>& layers = network->get_layers();
    const vector<vector<Index>>& input_indices = network->get_layer_input_indices();
    const Index B = batch_size;
    const type* last = nullptr;
    last_output_is_logits = false;

    // Padding flags of this position's keys, one row of B bytes per position in each self-attention cache.  Where the
    // layer's input comes from an Embedding or a Normalization3d, that kernel writes the flags as it writes the rows
    // (the training path takes them from the same place); any other producer is scanned by the attention branch below.
    vector<uint8_t*> flags_from_producer(layers.size(), nullptr);
    vector<char> flags_are_written(layers.size(), 0);
    for(size_t i = 0; i < layers.size(); i++)
    {
        const MultiHeadAttention* attention = dynamic_cast<const MultiHeadAttention*>(layers[i].get());
        if(!attention || !decoder_side[i] || attention->is_cross_attention()) continue;
        const Index producer = input_indices[i][0];
        if(producer < 0 || flags_from_producer[size_t(producer)]) continue;
        const string& kind = layers[size_t(producer)]->get_name();
        if(kind != "Embedding" && kind != "Normalization3d") continue;
        flags_from_producer[size_t(producer)] = reinterpret_cast<uint8_t*>(caches[i]->key_is_pad.data) + position * B;
        flags_are_written[i] = 1;
    }

    // the current position's ids, one per sample, contiguous
    check_cuda(cudaMemcpy2DAsync(step_ids.data, sizeof(type), ids + position, size_t(ids_stride) * sizeof(type), sizeof(type), size_t(B),
                                 cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream())), "IncrementalDecoder: ids");

    auto input_of = [&](size_t layer, size_t port) -> const type*
    {
        const Index source = input_indices[layer][port];
        if(source < 0 || !decoder_side[size_t(source)]) throw std::runtime_error("IncrementalDecoder: unexpected wiring");
        return outputs[size_t(source)]->data;
    };

    for(size_t i = 0; i < layers.size(); i++)
    {
        if(!decoder_side[i]) continue;
        Layer* layer = layers[i].get();
        type* out = outputs[i]->data;

        if(Embedding* embedding = dynamic_cast<Embedding*>(layer))
        {
            if(!embedding->positional_encoding_device.data) embedding->copy_positional_encoding_device();
            const Index E = embedding->embedding_dimension;
            check_onn(onn_embedding_fwd(step_ids.data, embedding->weights_device.data, embedding->positional_encoding_device.data + position * E, out,
                                        flags_from_producer[i], B, 1, E, embedding->vocabulary_size, embedding->scale_embedding,
                                        embedding->add_positional_encoding, 0, stream()), "IncrementalDecoder: embedding");
        }
        else if(MultiHeadAttention* attention = dynamic_cast<MultiHeadAttention*>(layer))
        {
            const Index E = attention->embedding_dimension, H = attention->heads_number;
            const type* x = input_of(i, 0);
            AttentionCache& cache = *caches[i];
            Index length = cache.capacity;                              // cross-attention: the whole encoder output
            if(attention->cross_attention)
                check_onn(onn_dense_fwd(x, attention->query_weights_device.data, attention->query_biases_device.data, query.data, nullptr,
                                        B, E, E, ONN_ACT_LINEAR, 0, stream()), "IncrementalDecoder: query");
            else
            {
                // query, and this position's key and value rows straight into slot `position` of the caches (row pitch
                // capacity * E per sample): three products over the same input, one launch
                const float* weights[3] = {attention->query_weights_device.data, attention->key_weights_device.data, attention->value_weights_device.data};
                const float* biases[3] = {attention->query_biases_device.data, attention->key_biases_device.data, attention->value_biases_device.data};
                float* results[3] = {query.data, cache.keys.data + position * E, cache.values.data + position * E};
                const int64_t pitches[3] = {E, cache.capacity * E, cache.capacity * E};
                check_onn(onn_dense_fwd_shared_input(x, weights, biases, results, pitches, 3, B, E, E, stream()), "IncrementalDecoder: projections");
                // padding flag of the new key: the layer's input row is all zero (a PAD token behind a finished sequence)
                if(!flags_are_written[i])
                    check_onn(onn_rows_are_zero(x, reinterpret_cast<uint8_t*>(cache.key_is_pad.data) + position * B, B, E, stream()),
                              "IncrementalDecoder: padding");
                length = position + 1;
            }
            // flags: [B, capacity] for the encoder output, one row of B per position for the self-attention cache
            check_onn(onn_decode_attention(query.data, cache.keys.data, cache.values.data, reinterpret_cast<const uint8_t*>(cache.key_is_pad.data),
                                           attention->cross_attention ? cache.capacity : 1, attention->cross_attention ? 1 : B,
                                           context.data, B, cache.capacity, length, E, H, stream()), "IncrementalDecoder: attention");
            check_onn(onn_dense_fwd(context.data, attention->projection_weights_device.data, attention->projection_biases_device.data, out, nullptr,
                                    B, E, E, ONN_ACT_LINEAR, 0, stream()), "IncrementalDecoder: output projection");
        }
        else if(Dense3d* dense = dynamic_cast<Dense3d*>(layer))
        {
            const bool defer = output_logits && i + 1 == layers.size() && dense->get_activation_code() == ONN_ACT_SOFTMAX;
            last_output_is_logits = defer;
            check_onn(onn_dense_fwd(input_of(i, 0), dense->weights_device.data, dense->biases_device.data, out, nullptr, B, dense->inputs_number,
                                    dense->neurons_number, dense->get_activation_code(), defer ? ONN_DEFER_SOFTMAX : 0, stream()),
                      "IncrementalDecoder: dense");
        }
        else if(Normalization3d* norm = dynamic_cast<Normalization3d*>(layer))
        {
            // statistics are not kept: inference only.  An Addition<3> that only this layer reads is summed inside the kernel
            const type* x = nullptr;
            const type* addend = nullptr;
            const Index source = input_indices[i][0];
            if(source >= 0 && forward_propagation->layers[size_t(source)]->fused_into_consumer)
            {
                x = input_of(size_t(source), 0);
                addend = input_of(size_t(source), 1);
            }
            else
                x = input_of(i, 0);
            check_onn(onn_layernorm_fwd(x, addend, norm->gammas_device.data, norm->betas_device.data, out, nullptr, query.data,
                                        query.data + B, flags_from_producer[i], B, norm->embedding_dimension, EPSILON, 0, stream()), "IncrementalDecoder: normalization");
        }
        else if(dynamic_cast<Addition3d*>(layer))
        {
            if(!forward_propagation->layers[i]->fused_into_consumer)
                check_onn(onn_add(input_of(i, 0), input_of(i, 1), out, outputs[i]->size(), 0, stream()), "IncrementalDecoder: addition");
        }
        else
            throw std::runtime_error("IncrementalDecoder: layer type " + layer->get_name() + " is not handled");
        last = out;
    }
    return last;
}

}  // namespace opennn_b200
