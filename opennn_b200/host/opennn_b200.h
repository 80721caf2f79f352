// C++ host mirror of the OpenNN interfaces on the transformer training path.  Class, method
// and member names follow OpenNN (opennn/layer.h, neural_network.h, loss.h,
// adaptive_moment_estimation.h) so that code written against OpenNN's `...Cuda` overloads
// reads the same here; every device computation goes through the C ABI of libonn_b200.so
// (include/onn_b200.h).  There is no CPU path: without a CUDA device the calls throw.
//
// What differs from OpenNN is decided once, when the propagation structures are set up
// (ForwardPropagationCuda::set / NeuralNetworkBackPropagationCuda::set), and never changes
// a layer's interface:
//   - an Addition<3> whose only consumer is a Normalization3d is computed inside that
//     layer's kernel (its `outputs` still receive the sum);
//   - gradients that fan in from several consumers are summed by the consuming kernel;
//   - a Dense "Linear" layer fed by a Dense "RectifiedLinear" layer applies the ReLU
//     derivative in its dX GEMM epilogue;
//   - the output layer's softmax is fused into CrossEntropyError3d while training.
#pragma once

#include <cuda_runtime.h>

#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/onn_b200.h"

namespace opennn_b200
{

using type = float;
using Index = long long;
using Shape = std::vector<Index>;
using std::string;
using std::unique_ptr;
using std::vector;

constexpr type EPSILON = 1.1920929e-07f;        // numeric_limits<float>::epsilon(), opennn/pch.h:123

void check_cuda(cudaError_t status, const char* what);
void check_onn(int status, const char* what);   // non-zero C-ABI status -> runtime_error (OpenNN's error convention)

// opennn/tensor_utilities.h:916-998 -- a non-owning device view
struct TensorViewCuda
{
    type* data = nullptr;
    Shape shape;

    TensorViewCuda() {}
    TensorViewCuda(type* new_data, const Shape& new_shape) : data(new_data), shape(new_shape) {}
    Index size() const;
};

// opennn/tensor_utilities.h:1001-1127 -- owning device buffer (cudaMalloc + memset)
struct TensorCuda
{
    type* data = nullptr;
    Index count = 0;
    Index capacity = 0;               // floats allocated: count rounded up to 1024, the slack zero-filled, so that a
                                      // collective may round an arena up to a multiple of 4 * ranks floats

    TensorCuda() {}
    ~TensorCuda() { free(); }
    TensorCuda(const TensorCuda&) = delete;
    TensorCuda& operator=(const TensorCuda&) = delete;

    void resize(Index new_count);
    void fill(type value);            // only 0 is supported (cudaMemsetAsync)
    void free();
    Index size() const { return count; }
};

// opennn/tensor_utilities.cpp:472-528, 650-703 -- arena packing, every view padded to 8 floats
Index get_size(const vector<TensorViewCuda*>& views);
Index get_size(const vector<vector<TensorViewCuda*>>& views);
type* link(type* pointer, const vector<TensorViewCuda*>& views);
void link(type* pointer, const vector<vector<TensorViewCuda*>>& views);

// opennn/tensor_utilities.h:841-868 -- process-wide device state (here: the compute stream)
class Device
{
public:
    static Device& instance();
    cudaStream_t get_compute_stream() const { return compute_stream; }
    void set_compute_stream(cudaStream_t stream) { compute_stream = stream; }
private:
    cudaStream_t compute_stream = nullptr;
};

class Layer;

// opennn/layer.h:457-490
struct LayerForwardPropagationCuda
{
    virtual ~LayerForwardPropagationCuda() = default;

    void set(Index new_batch_size, Layer* new_layer);
    virtual void initialize() = 0;
    virtual vector<TensorViewCuda*> get_workspace_views();
    TensorViewCuda get_outputs() const { return outputs; }

    Index batch_size = 0;
    Layer* layer = nullptr;
    vector<TensorViewCuda> inputs;
    TensorViewCuda outputs;

    // set-up time plan (see the header comment)
    TensorViewCuda outputs_row_is_zero;     // [rows] bytes packed in floats; produced when a consumer needs key-padding flags
    bool wants_row_flags = false;
    bool fused_into_consumer = false;       // Addition<3> computed by the following Normalization3d
};

// opennn/layer.h:492-528
struct LayerBackPropagationCuda
{
    virtual ~LayerBackPropagationCuda() = default;

    void set(Index new_batch_size, Layer* new_layer);
    virtual void initialize() = 0;
    virtual vector<TensorViewCuda*> get_gradient_views() { return {}; }
    virtual vector<TensorViewCuda*> get_workspace_views();
    vector<TensorViewCuda> get_input_gradients() const { return input_gradients; }

    Index batch_size = 0;
    Layer* layer = nullptr;
    vector<TensorViewCuda> input_gradients;
    vector<TensorViewCuda> output_gradients;

    // set-up time plan
    bool fused_into_consumer = false;       // Addition<3>: both input gradients alias the consumer's
    vector<bool> accumulate_input_gradient; // per port: add into a buffer shared with other consumers
    vector<bool> owns_input_gradient;       // per port: false when the view aliases another layer's buffer
};

// opennn/layer.h:32-376 -- the part of Layer the transformer path uses
class Layer
{
public:
    virtual ~Layer() = default;

    const string& get_name() const { return name; }
    const string& get_label() const { return label; }
    void set_label(const string& new_label) { label = new_label; }

    virtual Shape get_input_shape() const = 0;
    virtual Shape get_output_shape() const = 0;
    virtual vector<TensorViewCuda*> get_parameter_views_device() { return {}; }
    Index get_parameters_number();

    virtual void set_parameters_random(vector<type>& host_parameters, Index offset, unsigned seed) const {}

    virtual void forward_propagate(unique_ptr<LayerForwardPropagationCuda>&, bool is_training) = 0;
    virtual void back_propagate(unique_ptr<LayerForwardPropagationCuda>&, unique_ptr<LayerBackPropagationCuda>&) const = 0;

    // OpenNN creates these through Registry<...>::create(get_name()) (opennn/registry.h); a virtual does the same job
    virtual unique_ptr<LayerForwardPropagationCuda> create_forward_propagation() const = 0;
    virtual unique_ptr<LayerBackPropagationCuda> create_back_propagation() const = 0;

protected:
    string name = "Layer";
    string label;
};


// ---------------------------------------------------------------------------------------
// Embedding (opennn/embedding_layer.h)
// ---------------------------------------------------------------------------------------

class IncrementalDecoder;

class Embedding final : public Layer
{
    friend class IncrementalDecoder;
public:
    Embedding(const Shape& input_shape = {0, 0}, Index embedding_dimension = 0, const string& label = "embedding_layer");

    Index get_vocabulary_size() const { return vocabulary_size; }
    Index get_sequence_length() const { return sequence_length; }
    Index get_embedding_dimension() const { return embedding_dimension; }
    Shape get_input_shape() const override { return {sequence_length}; }
    Shape get_output_shape() const override { return {sequence_length, embedding_dimension}; }
    vector<TensorViewCuda*> get_parameter_views_device() override { return {&weights_device}; }

    void set(Index vocabulary_size, Index sequence_length, Index embedding_dimension, const string& label = "embedding_layer");
    void set_scale_embedding(bool value) { scale_embedding = value; }
    void set_add_positional_encoding(bool value) { add_positional_encoding = value; }
    void set_parameters_random(vector<type>&, Index, unsigned) const override;
    void copy_positional_encoding_device();            // opennn/embedding_layer.cpp:408-417
    const vector<type>& get_positional_encoding() const { return positional_encoding; }

    void forward_propagate(unique_ptr<LayerForwardPropagationCuda>&, bool) override;
    void back_propagate(unique_ptr<LayerForwardPropagationCuda>&, unique_ptr<LayerBackPropagationCuda>&) const override;
    unique_ptr<LayerForwardPropagationCuda> create_forward_propagation() const override;
    unique_ptr<LayerBackPropagationCuda> create_back_propagation() const override;

private:
    Index vocabulary_size = 0, sequence_length = 0, embedding_dimension = 0;
    bool scale_embedding = false, add_positional_encoding = false;
    vector<type> positional_encoding;                  // built on the host, opennn/embedding_layer.cpp:74-85
    TensorCuda positional_encoding_device;
    TensorViewCuda weights_device;
};

struct EmbeddingForwardPropagationCuda final : LayerForwardPropagationCuda
{
    void initialize() override;
};

struct EmbeddingBackPropagationCuda final : LayerBackPropagationCuda
{
    void initialize() override;
    vector<TensorViewCuda*> get_gradient_views() override { return {&weight_gradients}; }
    TensorViewCuda weight_gradients;
};


// ---------------------------------------------------------------------------------------
// MultiHeadAttention (opennn/multihead_attention_layer.h)
// ---------------------------------------------------------------------------------------

class MultiHeadAttention final : public Layer
{
    friend class IncrementalDecoder;
public:
    MultiHeadAttention(const Shape& query_shape = {0, 0}, Index heads_number = 0, const string& label = "multihead_attention_layer");
    MultiHeadAttention(const Shape& query_shape, const Shape& source_shape, Index heads_number, const string& label = "multihead_attention_layer");

    void set(Index query_sequence_length, Index source_sequence_length, Index embedding_dimension, Index heads_number,
             bool use_causal_mask, const string& label = "multihead_attention_layer");

    Index get_query_sequence_length() const { return query_sequence_length; }
    Index get_source_sequence_length() const { return source_sequence_length; }
    Index get_embedding_dimension() const { return embedding_dimension; }
    Index get_heads_number() const { return heads_number; }
    Index get_head_dimension() const { return heads_number ? embedding_dimension / heads_number : 0; }
    bool get_use_causal_mask() const { return use_causal_mask; }
    bool is_cross_attention() const { return cross_attention; }
    Shape get_input_shape() const override { return {query_sequence_length, embedding_dimension}; }
    Shape get_output_shape() const override { return {query_sequence_length, embedding_dimension}; }

    vector<TensorViewCuda*> get_parameter_views_device() override;       // {Wq,bq,Wk,bk,Wv,bv,Wo,bo}: multihead_attention_layer.cpp:105-108
    void set_parameters_random(vector<type>&, Index, unsigned) const override;

    void forward_propagate(unique_ptr<LayerForwardPropagationCuda>&, bool) override;
    void back_propagate(unique_ptr<LayerForwardPropagationCuda>&, unique_ptr<LayerBackPropagationCuda>&) const override;
    unique_ptr<LayerForwardPropagationCuda> create_forward_propagation() const override;
    unique_ptr<LayerBackPropagationCuda> create_back_propagation() const override;

private:
    Index query_sequence_length = 0, source_sequence_length = 0, embedding_dimension = 0, heads_number = 0;
    bool use_causal_mask = false, cross_attention = false;
    TensorViewCuda query_weights_device, query_biases_device, key_weights_device, key_biases_device,
                   value_weights_device, value_biases_device, projection_weights_device, projection_biases_device;
};

struct MultiHeadAttentionForwardPropagationCuda final : LayerForwardPropagationCuda
{
    void initialize() override;
    vector<TensorViewCuda*> get_workspace_views() override;
    TensorViewCuda attention_state;          // Q, K, V, attention weights, concatenated head outputs (one C-ABI workspace)
    const uint8_t* source_row_is_zero = nullptr;
};

struct MultiHeadAttentionBackPropagationCuda final : LayerBackPropagationCuda
{
    void initialize() override;
    vector<TensorViewCuda*> get_gradient_views() override;
    TensorViewCuda query_weight_gradients, query_bias_gradients, key_weight_gradients, key_bias_gradients,
                   value_weight_gradients, value_bias_gradients, projection_weight_gradients, projection_bias_gradients;
    TensorViewCuda scratch;                  // shared by all attention layers (NeuralNetworkBackPropagationCuda owns it)
    Index scratch_floats = 0;
    bool projection_bias_gradient_is_ready = false;   // taken by the following Normalization3d as column sums of its dx
};


// ---------------------------------------------------------------------------------------
// Dense<3> (opennn/dense_layer.h)
// ---------------------------------------------------------------------------------------

class Dense3d final : public Layer
{
    friend class IncrementalDecoder;
public:
    Dense3d(Index sequence_length, Index input_features, Index neurons, const string& activation, const string& label);
    // Dense<2> (opennn/dense_layer.h with Rank = 2): the same layer on [batch, features] rows; it reports the name
    // "Dense2d" as the reference does, and takes no part in the set-up plans written for the transformer's Dense3d pairs
    static unique_ptr<Dense3d> make_rank2(Index input_features, Index neurons, const string& activation, const string& label);

    Index get_sequence_length() const { return sequence_length; }
    Index get_input_features_number() const { return inputs_number; }
    Index get_neurons_number() const { return neurons_number; }
    const string& get_activation_function() const { return activation_function; }
    int get_activation_code() const;
    Shape get_input_shape() const override { return {sequence_length, inputs_number}; }
    Shape get_output_shape() const override { return {sequence_length, neurons_number}; }

    vector<TensorViewCuda*> get_parameter_views_device() override { return {&biases_device, &weights_device}; }  // dense_layer.h:484
    void set_parameters_random(vector<type>&, Index, unsigned) const override;

    void forward_propagate(unique_ptr<LayerForwardPropagationCuda>&, bool) override;
    void back_propagate(unique_ptr<LayerForwardPropagationCuda>&, unique_ptr<LayerBackPropagationCuda>&) const override;
    unique_ptr<LayerForwardPropagationCuda> create_forward_propagation() const override;
    unique_ptr<LayerBackPropagationCuda> create_back_propagation() const override;

private:
    Index sequence_length = 0, inputs_number = 0, neurons_number = 0;
    string activation_function = "Linear";
    TensorViewCuda biases_device, weights_device;
};

struct Dense3dForwardPropagationCuda final : LayerForwardPropagationCuda
{
    void initialize() override;
    vector<TensorViewCuda*> get_workspace_views() override;
    bool defer_softmax = false;              // training with CrossEntropyError3d: outputs hold logits
    TensorViewCuda relu_bits;                // (outputs > 0) at one bit per element, 32-bit words held in a float view
    bool wants_relu_bits = false;            // the only consumer is a Dense3d whose dX epilogue applies this layer's ReLU derivative
};

struct Dense3dBackPropagationCuda final : LayerBackPropagationCuda
{
    void initialize() override;
    vector<TensorViewCuda*> get_gradient_views() override { return {&bias_gradients, &weight_gradients}; }   // dense_layer.h:107
    TensorViewCuda bias_gradients, weight_gradients;
    bool delta_is_ready = false;             // the consumer's dX epilogue already applied this layer's ReLU derivative
    const type* input_relu_mask = nullptr;   // outputs of the ReLU layer that produced this layer's input
    const uint32_t* input_relu_bits = nullptr;   // the same mask as bits, written by that layer's forward pass
    bool skip_input_gradient = false;
    type* input_bias_gradients = nullptr;    // bias gradients of that ReLU layer: column sums of this layer's dX
    bool bias_gradient_is_ready = false;     // the consumer's dX epilogue already accumulated this layer's bias gradient
};


// ---------------------------------------------------------------------------------------
// Normalization3d (opennn/normalization_layer_3d.h) and Addition<3> (opennn/addition_layer.h)
// ---------------------------------------------------------------------------------------

class Normalization3d final : public Layer
{
    friend class IncrementalDecoder;
public:
    Normalization3d(const Shape& input_shape = {0, 0}, const string& label = "normalization_layer_3d");

    Index get_sequence_length() const { return sequence_length; }
    Index get_embedding_dimension() const { return embedding_dimension; }
    Shape get_input_shape() const override { return {sequence_length, embedding_dimension}; }
    Shape get_output_shape() const override { return {sequence_length, embedding_dimension}; }
    vector<TensorViewCuda*> get_parameter_views_device() override { return {&gammas_device, &betas_device}; }  // normalization_layer_3d.cpp:49
    void set_parameters_random(vector<type>&, Index, unsigned) const override;

    void forward_propagate(unique_ptr<LayerForwardPropagationCuda>&, bool) override;
    void back_propagate(unique_ptr<LayerForwardPropagationCuda>&, unique_ptr<LayerBackPropagationCuda>&) const override;
    unique_ptr<LayerForwardPropagationCuda> create_forward_propagation() const override;
    unique_ptr<LayerBackPropagationCuda> create_back_propagation() const override;

private:
    Index sequence_length = 0, embedding_dimension = 0;
    TensorViewCuda gammas_device, betas_device;
};

struct Normalization3dForwardPropagationCuda final : LayerForwardPropagationCuda
{
    void initialize() override;
    vector<TensorViewCuda*> get_workspace_views() override;
    TensorViewCuda means, inverse_standard_deviations;
    // fused Addition<3>: the two addends and where the sum goes (the Addition layer's outputs)
    const type* addend_a = nullptr;
    const type* addend_b = nullptr;
    type* sum_output = nullptr;
};

struct Normalization3dBackPropagationCuda final : LayerBackPropagationCuda
{
    void initialize() override;
    vector<TensorViewCuda*> get_gradient_views() override { return {&gamma_gradients, &beta_gradients}; }     // normalization_layer_3d.cpp:320
    vector<TensorViewCuda*> get_workspace_views() override;
    TensorViewCuda gamma_gradients, beta_gradients;
    TensorViewCuda partial_sums;
    type* input_bias_gradients = nullptr;    // bias gradient of the layer whose output gradient is this layer's input gradient
};

class Addition3d final : public Layer
{
public:
    Addition3d(const Shape& input_shape = {0, 0}, const string& label = "addition_layer");
    Shape get_input_shape() const override { return {sequence_length, embedding_dimension}; }
    Shape get_output_shape() const override { return {sequence_length, embedding_dimension}; }

    void forward_propagate(unique_ptr<LayerForwardPropagationCuda>&, bool) override;
    void back_propagate(unique_ptr<LayerForwardPropagationCuda>&, unique_ptr<LayerBackPropagationCuda>&) const override;
    unique_ptr<LayerForwardPropagationCuda> create_forward_propagation() const override;
    unique_ptr<LayerBackPropagationCuda> create_back_propagation() const override;

private:
    Index sequence_length = 0, embedding_dimension = 0;
};

struct Addition3dForwardPropagationCuda final : LayerForwardPropagationCuda
{
    void initialize() override;
};

struct Addition3dBackPropagationCuda final : LayerBackPropagationCuda
{
    void initialize() override;
};


// ---------------------------------------------------------------------------------------
// Pooling3d (opennn/pooling_layer_3d.h): pooling over the sequence in front of a classification head
// ---------------------------------------------------------------------------------------

class Pooling3d final : public Layer
{
public:
    enum class PoolingMethod { MaxPooling, AveragePooling };
    Pooling3d(const Shape& input_shape = {0, 0}, PoolingMethod method = PoolingMethod::MaxPooling, const string& label = "sequence_pooling_layer");
    PoolingMethod get_pooling_method() const { return pooling_method; }
    Shape get_input_shape() const override { return {sequence_length, features}; }
    Shape get_output_shape() const override { return {features}; }

    void forward_propagate(unique_ptr<LayerForwardPropagationCuda>&, bool) override;
    void back_propagate(unique_ptr<LayerForwardPropagationCuda>&, unique_ptr<LayerBackPropagationCuda>&) const override;
    unique_ptr<LayerForwardPropagationCuda> create_forward_propagation() const override;
    unique_ptr<LayerBackPropagationCuda> create_back_propagation() const override;

private:
    Index sequence_length = 0, features = 0;
    PoolingMethod pooling_method = PoolingMethod::MaxPooling;
};

struct Pooling3dForwardPropagationCuda final : LayerForwardPropagationCuda
{
    void initialize() override;
    vector<TensorViewCuda*> get_workspace_views() override;
    TensorViewCuda maximal_indices;          // int32 [batch, features], held in a float view
    TensorViewCuda row_is_valid;             // bytes [batch * sequence], held in a float view
    TensorViewCuda valid_count;              // int32 [batch]
};

struct Pooling3dBackPropagationCuda final : LayerBackPropagationCuda
{
    void initialize() override;
};

// ---------------------------------------------------------------------------------------
// NeuralNetwork (opennn/neural_network.h) and the Transformer builder (opennn/standard_networks.h)
// ---------------------------------------------------------------------------------------

struct ForwardPropagationCuda;

class NeuralNetwork
{
public:
    virtual ~NeuralNetwork() = default;

    void add_layer(unique_ptr<Layer> layer, const vector<Index>& input_indices = {});   // neural_network.h:84
    void compile();                                                                    // neural_network.cpp:66-94

    Index get_layers_number() const { return Index(layers.size()); }
    const vector<unique_ptr<Layer>>& get_layers() const { return layers; }
    const vector<vector<Index>>& get_layer_input_indices() const { return layer_input_indices; }
    vector<vector<Index>> get_layer_output_indices() const;
    Index find_input_index(const vector<Index>& indices, Index layer_index) const;
    Index get_first_trainable_layer_index() const { return 0; }
    Index get_last_trainable_layer_index() const { return get_layers_number() - 1; }
    Index get_parameters_number() const { return Index(parameters.size()); }
    Shape get_output_shape() const { return layers.back()->get_output_shape(); }

    vector<type>& get_parameters() { return parameters; }
    void set_parameters_random(unsigned seed = 0);
    void copy_parameters_device();                 // host -> device arena
    void copy_parameters_host();                   // device -> host

    TensorCuda& get_parameters_device() { return parameters_device; }

    // neural_network.cpp:1889-1943.  input_views: {decoder ids, encoder ids} for the Transformer
    // (external input -1 = first, -2 = second: standard_networks.cpp:669-704).
    // run_layer (optional, one flag per layer): layers whose flag is 0 keep the outputs of an earlier pass -- the decoding
    // loop runs the encoder side once and only the layers that depend on the decoder ids afterwards
    void forward_propagate(const vector<TensorViewCuda>& input_views, ForwardPropagationCuda& forward_propagation, bool is_training,
                           const vector<char>* run_layer = nullptr);
    // 1 for every layer whose output depends on external input number `external` (1 = decoder ids, 2 = encoder ids)
    vector<char> layers_depending_on_input(Index external) const;

    // Called before each layer's forward pass (no counterpart in OpenNN): the data-parallel trainer makes the compute
    // stream wait here for the all-gather that brings this layer's updated parameters, so that the gathers of the later
    // layers run under the forward pass of the earlier ones.
    void (*before_layer_hook)(void* context, Index layer) = nullptr;
    void* before_layer_context = nullptr;

protected:
    vector<unique_ptr<Layer>> layers;
    vector<vector<Index>> layer_input_indices;
    vector<type> parameters;
    TensorCuda parameters_device;
};

class Transformer final : public NeuralNetwork
{
public:
    // standard_networks.cpp:638-907: post-norm encoder-decoder, 2 + 7L + 10L + 1 layers
    Transformer(Index input_sequence_length, Index decoder_sequence_length, Index input_vocabulary_size,
                Index output_vocabulary_size, Index embedding_dimension, Index heads_number,
                Index feed_forward_dimension, Index layers_number);
};

// standard_networks.cpp:575-615: Embedding (scaled, with positions) -> self-attention -> max pooling over the sequence ->
// Dense<2> "RectifiedLinear" layers -> Dense<2> "Softmax" (more than one class)
class TextClassificationNetwork final : public NeuralNetwork
{
public:
    TextClassificationNetwork(Index vocabulary_size, Index sequence_length, Index embedding_dimension, Index heads_number,
                              const vector<Index>& complexity_dimensions, Index classes);
};

// Decoder-only stack assembled with add_layer the way Transformer assembles its decoder,
// minus cross-attention.
unique_ptr<NeuralNetwork> make_decoder_only_network(Index sequence_length, Index vocabulary_size, Index embedding_dimension,
                                                    Index heads_number, Index feed_forward_dimension, Index layers_number);

// neural_network.h:28-79
struct ForwardPropagationCuda
{
    ForwardPropagationCuda(Index samples_number = 0, NeuralNetwork* neural_network = nullptr);
    void set(Index samples_number, NeuralNetwork* neural_network);
    TensorViewCuda get_last_trainable_layer_outputs_device() const { return layers.back()->outputs; }
    TensorViewCuda get_outputs() { return layers.back()->outputs; }

    Index samples_number = 0;
    NeuralNetwork* neural_network = nullptr;
    vector<unique_ptr<LayerForwardPropagationCuda>> layers;
    TensorCuda workspace;
};

// neural_network.h:316-342
struct NeuralNetworkBackPropagationCuda
{
    void set(Index batch_size, NeuralNetwork* neural_network, ForwardPropagationCuda* forward_propagation);

    Index batch_size = 0;
    NeuralNetwork* neural_network = nullptr;
    vector<unique_ptr<LayerBackPropagationCuda>> layers;
    TensorCuda gradients;             // one arena, same layer order and padding as the parameters
    TensorCuda workspace;
    TensorCuda attention_scratch;     // transient back-propagation buffers shared by all attention layers
};


// ---------------------------------------------------------------------------------------
// CrossEntropyError3d (opennn/cross_entropy_error_3d.h, opennn/loss.h)
// ---------------------------------------------------------------------------------------

// dataset.h:560-618 BatchCuda, reduced to what the path reads: device views of the ids and targets
struct BatchCuda
{
    TensorViewCuda decoder;           // [B, S_dec] floats holding integers (first external input)
    TensorViewCuda input;             // [B, S_in]  (second external input; empty for decoder-only)
    TensorViewCuda target;            // [B, S_dec]
    Index samples_number = 0;

    vector<TensorViewCuda> get_inputs_device() const;          // {decoder, input}: dataset.cpp:4331-4339
    TensorViewCuda get_targets_device() const { return target; }
    bool is_empty() const { return samples_number == 0; }
};

class CrossEntropyError3d;

// loss.h:283-317
struct BackPropagationCuda
{
    BackPropagationCuda(Index samples_number = 0, CrossEntropyError3d* loss = nullptr, ForwardPropagationCuda* forward_propagation = nullptr);
    void set(Index samples_number, CrossEntropyError3d* loss, ForwardPropagationCuda* forward_propagation);
    TensorViewCuda get_output_gradients_device() const { return output_gradients; }

    Index samples_number = 0;
    CrossEntropyError3d* loss = nullptr;
    NeuralNetworkBackPropagationCuda neural_network;

    type error = 0;                   // filled by read_error()
    type accuracy = 0;
    type loss_value = 0;

    TensorViewCuda output_gradients;  // aliases the output layer's buffer: the fused kernel writes the gradient in place
    TensorCuda statistics;            // {sum of -log terms, #correct, #active (this batch), 0} x accumulation slots
    Index statistics_slot = 0;        // slots filled since the last read_error
    TensorCuda active_count;          // #active tokens the gradient is scaled by (global batch)
    TensorCuda row_scratch;
    type* pinned_statistics = nullptr;
    ~BackPropagationCuda();
};

class CrossEntropyError3d
{
public:
    explicit CrossEntropyError3d(NeuralNetwork* neural_network = nullptr) : neural_network(neural_network) {}
    NeuralNetwork* get_neural_network() const { return neural_network; }
    void set_regularization_method(const string& method);      // only "None" is implemented (loss.h:197-199 default is L2)

    // cross_entropy_error_3d.cpp:370-454: counts the active targets of `batch` into back_propagation.active_count
    void calculate_active_tokens(const BatchCuda& batch, BackPropagationCuda& back_propagation) const;
    // cross_entropy_error_3d.cpp:370-454 + 498-528 in one kernel: loss statistics and output gradients
    void calculate_error_and_output_gradients(const BatchCuda& batch, ForwardPropagationCuda& forward_propagation,
                                              BackPropagationCuda& back_propagation, bool accumulate_statistics) const;
    // loss.cpp:1249-1289: error -> output gradients -> reverse layer walk.  No host synchronisation.
    void back_propagate(const BatchCuda& batch, ForwardPropagationCuda& forward_propagation, BackPropagationCuda& back_propagation,
                        bool accumulate_statistics = false) const;
    void calculate_layers_error_gradient(ForwardPropagationCuda& forward_propagation, BackPropagationCuda& back_propagation) const;
    // one small D2H read of the statistics (the reference blocks twice per step: cross_entropy_error_3d.cpp:424, 435)
    void read_error(BackPropagationCuda& back_propagation, type global_active_tokens = 0) const;

    // a hook the data-parallel driver sets: called once the gradients of layers >= first_layer are final
    void (*gradient_ready_hook)(void* context, Index first_layer) = nullptr;
    void* gradient_ready_context = nullptr;

private:
    NeuralNetwork* neural_network = nullptr;
    string regularization_method = "None";
};


// ---------------------------------------------------------------------------------------
// AdaptiveMomentEstimation (opennn/adaptive_moment_estimation.h)
// ---------------------------------------------------------------------------------------

// CrossEntropyError2d with several classes (opennn/cross_entropy_error.cpp:58-77, 114-134, CUDA :217-300): the loss
// of a classification head whose last layer is a Dense<2> "Softmax".  error = -sum(t log(y + eps)) / samples; the
// output gradient (y - t) / samples replaces the probabilities in the last layer's output buffer and goes through
// that layer's back-propagation unchanged.
class CrossEntropyError2d
{
public:
    explicit CrossEntropyError2d(NeuralNetwork* network = nullptr) : neural_network(network) {}
    NeuralNetwork* get_neural_network() const { return neural_network; }
    // targets [samples, classes]; statistics (device, 2 floats) receives {error, samples}; row_scratch [samples]
    void back_propagate(const TensorViewCuda& targets, ForwardPropagationCuda& forward_propagation,
                        NeuralNetworkBackPropagationCuda& back_propagation, type* statistics, type* row_scratch) const;
private:
    NeuralNetwork* neural_network = nullptr;
};

class AdaptiveMomentEstimation;

// adaptive_moment_estimation.h:139-160
struct ADAMOptimizationDataCuda
{
    explicit ADAMOptimizationDataCuda(AdaptiveMomentEstimation* optimizer = nullptr);
    void set(AdaptiveMomentEstimation* optimizer);
    void set(Index parameters_number);

    AdaptiveMomentEstimation* adaptive_moment_estimation = nullptr;
    TensorCuda gradient_exponential_decay;           // m
    TensorCuda square_gradient_exponential_decay;    // v
    TensorCuda square_norm;                          // ||g||^2 on the device
    TensorCuda norm_workspace;
    Index iteration = 1;                             // starts at 1, incremented before use: adaptive_moment_estimation.cpp:233, 449
};

class AdaptiveMomentEstimation
{
public:
    explicit AdaptiveMomentEstimation(CrossEntropyError3d* loss = nullptr) : loss(loss) {}
    CrossEntropyError3d* get_loss() const { return loss; }
    void set_learning_rate(type value) { learning_rate = value; }
    void set_beta_1(type value) { beta_1 = value; }
    void set_beta_2(type value) { beta_2 = value; }
    void set_gradient_clip_norm(type value) { gradient_clip_norm = value; }
    type get_learning_rate() const { return learning_rate; }

    // adaptive_moment_estimation.cpp:855-883 with the CPU path's global-norm clip (:462-466).
    // gradient_scale multiplies the gradient first (1 unless the caller averaged an all-reduce).
    void update_parameters(BackPropagationCuda& back_propagation, ADAMOptimizationDataCuda& optimization_data,
                           type gradient_scale = 1) const;
    // the same update on any network and gradient arena (used with CrossEntropyError2d)
    void update_parameters(NeuralNetwork* network, TensorCuda& gradients, ADAMOptimizationDataCuda& optimization_data,
                           type gradient_scale = 1) const;
    // iteration++ and the two bias corrections of that iteration (adaptive_moment_estimation.cpp:449-454)
    void advance(ADAMOptimizationDataCuda& optimization_data, type& bias_correction_1, type& bias_correction_2) const;
    type get_beta_1() const { return beta_1; }
    type get_beta_2() const { return beta_2; }
    type get_gradient_clip_norm() const { return gradient_clip_norm; }
    // device word (or nullptr): when it is not zero the update kernel leaves parameters, moments and gradient alone
    // (onn_adam_guarded): a step whose kernels gave up on a bounded wait must not reach the parameters
    void set_skip_word(const uint32_t* word) { skip_if_nonzero = word; }

private:
    CrossEntropyError3d* loss = nullptr;
    type learning_rate = type(0.001), beta_1 = type(0.9), beta_2 = type(0.999), gradient_clip_norm = type(1.0);   // .h:86-92
    const uint32_t* skip_if_nonzero = nullptr;
};


// ---------------------------------------------------------------------------------------
// Decoding one token at a time with cached keys and values.  Transformer::calculate_outputs
// (opennn/standard_networks.cpp:1002-1035) runs the whole network on the whole target for every new
// token; here the encoder side runs once, each decoder-side layer sees ONE position per step
// ([batch, 1, features]), self-attention layers append that position's key and value rows to a
// cache and attend over it (causality is what the cache holds), cross-attention layers attend over
// keys and values projected once from the encoder output.
// ---------------------------------------------------------------------------------------

class IncrementalDecoder
{
public:
    IncrementalDecoder(NeuralNetwork* network, ForwardPropagationCuda* forward_propagation, Index batch_size);

    // After the encoder side has been run by NeuralNetwork::forward_propagate (its outputs are in
    // forward_propagation): projects the cross-attention keys and values and clears the self-attention caches.
    void start();
    // Feeds the decoder ids of `position` (device, one float per sample at ids[b * ids_stride + position]) through the
    // decoder side and returns the device pointer of the last layer's output for that position: [batch, vocabulary].
    // output_logits: if the last layer is a Dense "Softmax", leave its logits (the caller fuses the softmax into what
    // it does next); true is returned through output_is_logits() for that step
    const type* step(const type* ids, Index ids_stride, Index position, bool output_logits = false);
    bool output_is_logits() const { return last_output_is_logits; }

private:
    struct AttentionCache { TensorCuda keys, values, key_is_pad; Index capacity = 0; };
    bool last_output_is_logits = false;

    NeuralNetwork* network = nullptr;
    ForwardPropagationCuda* forward_propagation = nullptr;
    Index batch_size = 0;
    vector<char> decoder_side;
    vector<unique_ptr<TensorCuda>> outputs;       // per decoder-side layer: [batch, width] of the current position
    vector<unique_ptr<AttentionCache>> caches;    // per decoder-side MultiHeadAttention layer
    TensorCuda query, context, step_ids;
};

}  // namespace opennn_b200
