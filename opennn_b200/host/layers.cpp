// Host mirror of OpenNN's transformer layers: every forward_propagate / back_propagate body
// is a handful of C-ABI calls (include/onn_b200.h) on the views the propagation structures
// hold.  See opennn_b200.h for what is decided at set-up time.
#include <cmath>
#include <cstring>
#include <random>

#include "opennn_b200.h"

namespace opennn_b200
{

// ---------------------------------------------------------------------------------------
// utilities (opennn/tensor_utilities.cpp)
// ---------------------------------------------------------------------------------------

void check_cuda(cudaError_t status, const char* what)
{
    if(status != cudaSuccess)
        throw std::runtime_error(string("CUDA Error: ") + cudaGetErrorString(status) + " in " + what);
}

void check_onn(int status, const char* what)
{
    if(status != ONN_OK)
        throw std::runtime_error(string(what) + ": " + onn_status_string(status));
}

Index TensorViewCuda::size() const
{
    if(shape.empty()) return 0;
    Index total = 1;
    for(const Index d : shape) total *= d;
    return total;
}

void TensorCuda::resize(Index new_count)
{
    free();
    if(new_count <= 0) return;
    capacity = (new_count + 1023) & ~Index(1023);
    check_cuda(cudaMalloc(reinterpret_cast<void**>(&data), size_t(capacity) * sizeof(type)), "TensorCuda::resize");
    count = new_count;
    check_cuda(cudaMemset(data, 0, size_t(capacity) * sizeof(type)), "TensorCuda::resize memset");
    // the fill runs on the legacy default stream and may return before it has run; the compute stream is non-blocking
    // and does not wait for it, so a kernel launched right after could see its output wiped
    check_cuda(cudaStreamSynchronize(nullptr), "TensorCuda::resize synchronize");
}

void TensorCuda::fill(type value)
{
    if(value != type(0)) throw std::runtime_error("TensorCuda::fill: only zero fill is implemented");
    if(count > 0)
        check_cuda(cudaMemsetAsync(data, 0, size_t(count) * sizeof(type), Device::instance().get_compute_stream()), "TensorCuda::fill");
}

void TensorCuda::free()
{
    if(data) cudaFree(data);
    data = nullptr;
    count = 0;
    capacity = 0;
}

static Index padded(Index count) { return (count + 7) & ~Index(7); }    // EIGEN_MAX_ALIGN_BYTES / sizeof(float) = 8

Index get_size(const vector<TensorViewCuda*>& views)
{
    Index total = 0;
    for(const TensorViewCuda* view : views)
        if(view && view->size() > 0) total += padded(view->size());
    return total;
}

Index get_size(const vector<vector<TensorViewCuda*>>& views)
{
    Index total = 0;
    for(const vector<TensorViewCuda*>& group : views) total += get_size(group);
    return total;
}

type* link(type* pointer, const vector<TensorViewCuda*>& views)
{
    for(TensorViewCuda* view : views)
    {
        if(!view || view->size() == 0) continue;
        if(reinterpret_cast<uintptr_t>(pointer) % 32 != 0) throw std::runtime_error("Master pointer in link() is not aligned.");
        view->data = pointer;
        pointer += padded(view->size());
    }
    return pointer;
}

void link(type* pointer, const vector<vector<TensorViewCuda*>>& views)
{
    for(const vector<TensorViewCuda*>& group : views) pointer = link(pointer, group);
}

Device& Device::instance()
{
    static Device device;
    return device;
}

static void* stream() { return Device::instance().get_compute_stream(); }

void LayerForwardPropagationCuda::set(Index new_batch_size, Layer* new_layer)
{
    if(!new_layer) return;
    batch_size = new_batch_size;
    layer = new_layer;
    initialize();
}

vector<TensorViewCuda*> LayerForwardPropagationCuda::get_workspace_views()
{
    vector<TensorViewCuda*> views = {&outputs};
    if(wants_row_flags) views.push_back(&outputs_row_is_zero);
    return views;
}

void LayerBackPropagationCuda::set(Index new_batch_size, Layer* new_layer)
{
    if(!new_layer) return;
    batch_size = new_batch_size;
    layer = new_layer;
    initialize();
    accumulate_input_gradient.assign(input_gradients.size(), false);
    owns_input_gradient.assign(input_gradients.size(), true);
}

vector<TensorViewCuda*> LayerBackPropagationCuda::get_workspace_views()
{
    vector<TensorViewCuda*> views;
    for(size_t i = 0; i < input_gradients.size(); i++)
        if(owns_input_gradient.empty() || owns_input_gradient[i]) views.push_back(&input_gradients[i]);
    return views;
}

Index Layer::get_parameters_number()
{
    return get_size(get_parameter_views_device());
}

static uint8_t* row_flags_of(LayerForwardPropagationCuda& forward)
{
    return forward.wants_row_flags ? reinterpret_cast<uint8_t*>(forward.outputs_row_is_zero.data) : nullptr;
}

// Sum of the consumer gradients that the kernels cannot take as extra operands (more than
// `direct` of them): folded into the first one with onn_add (opennn/layer.cpp:447-457).
static void fold_extra_gradients(const vector<TensorViewCuda>& gradients, size_t direct)
{
    for(size_t i = direct; i < gradients.size(); i++)
        check_onn(onn_add(gradients[0].data, gradients[i].data, gradients[0].data, gradients[0].size(), 0, stream()), "add_gradients");
}


// ---------------------------------------------------------------------------------------
// Embedding
// ---------------------------------------------------------------------------------------

Embedding::Embedding(const Shape& input_shape, Index new_embedding_dimension, const string& new_label)
{
    name = "Embedding";
    set(input_shape[0], input_shape[1], new_embedding_dimension, new_label);
}

void Embedding::set(Index new_vocabulary_size, Index new_sequence_length, Index new_embedding_dimension, const string& new_label)
{
    vocabulary_size = new_vocabulary_size;
    sequence_length = new_sequence_length;
    embedding_dimension = new_embedding_dimension;
    label = new_label;
    weights_device.shape = {vocabulary_size, embedding_dimension};

    // opennn/embedding_layer.cpp:74-85: first half sines, second half cosines; the exponent is a
    // float division, pow / sin / cos run in double, the table is stored as float
    positional_encoding.assign(size_t(sequence_length * embedding_dimension), type(0));
    const type half_depth = type(embedding_dimension) / 2;
    for(Index i = 0; i < sequence_length; i++)
        for(Index j = 0; j < embedding_dimension; j++)
            positional_encoding[size_t(i * embedding_dimension + j)] = (j < Index(half_depth))
                ? type(std::sin(i / std::pow(10000, j / half_depth)))
                : type(std::cos(i / std::pow(10000, (j - Index(half_depth)) / half_depth)));
}

void Embedding::copy_positional_encoding_device()
{
    if(positional_encoding.empty()) return;
    positional_encoding_device.resize(Index(positional_encoding.size()));
    check_cuda(cudaMemcpy(positional_encoding_device.data, positional_encoding.data(), positional_encoding.size() * sizeof(type),
                          cudaMemcpyHostToDevice), "copy_positional_encoding_device");
    check_cuda(cudaDeviceSynchronize(), "copy_positional_encoding_device");
}

void Embedding::set_parameters_random(vector<type>& host, Index offset, unsigned seed) const
{
    // opennn/embedding_layer.cpp:114-126: 0.05 * U(-1, 1), padding row zero
    std::mt19937 generator(seed);
    std::uniform_real_distribution<type> uniform(type(-1), type(1));
    for(Index i = 0; i < vocabulary_size * embedding_dimension; i++)
        host[size_t(offset + i)] = i < embedding_dimension ? type(0) : type(0.05) * uniform(generator);
}

void EmbeddingForwardPropagationCuda::initialize()
{
    const Embedding* embedding = static_cast<const Embedding*>(layer);
    outputs.shape = {batch_size, embedding->get_sequence_length(), embedding->get_embedding_dimension()};
    outputs_row_is_zero.shape = {(batch_size * embedding->get_sequence_length() + 3) / 4};
}

void EmbeddingBackPropagationCuda::initialize()
{
    const Embedding* embedding = static_cast<const Embedding*>(layer);
    weight_gradients.shape = {embedding->get_vocabulary_size(), embedding->get_embedding_dimension()};
    input_gradients.clear();                      // token ids carry no gradient
}

unique_ptr<LayerForwardPropagationCuda> Embedding::create_forward_propagation() const { return std::make_unique<EmbeddingForwardPropagationCuda>(); }
unique_ptr<LayerBackPropagationCuda> Embedding::create_back_propagation() const { return std::make_unique<EmbeddingBackPropagationCuda>(); }

void Embedding::forward_propagate(unique_ptr<LayerForwardPropagationCuda>& forward, bool)
{
    if(!positional_encoding_device.data) copy_positional_encoding_device();
    check_onn(onn_embedding_fwd(forward->inputs[0].data, weights_device.data, positional_encoding_device.data,
                                forward->outputs.data, row_flags_of(*forward), forward->batch_size, sequence_length,
                                embedding_dimension, vocabulary_size, scale_embedding, add_positional_encoding, 0, stream()),
              "Embedding::forward_propagate");
}

void Embedding::back_propagate(unique_ptr<LayerForwardPropagationCuda>& forward, unique_ptr<LayerBackPropagationCuda>& back) const
{
    EmbeddingBackPropagationCuda* this_back = static_cast<EmbeddingBackPropagationCuda*>(back.get());
    const vector<TensorViewCuda>& gradients = back->output_gradients;
    fold_extra_gradients(gradients, 2);
    check_onn(onn_embedding_bwd(forward->inputs[0].data, gradients[0].data, gradients.size() > 1 ? gradients[1].data : nullptr,
                                this_back->weight_gradients.data, forward->batch_size, sequence_length, embedding_dimension,
                                vocabulary_size, scale_embedding, stream()),
              "Embedding::back_propagate");
}


// ---------------------------------------------------------------------------------------
// MultiHeadAttention
// ---------------------------------------------------------------------------------------

MultiHeadAttention::MultiHeadAttention(const Shape& query_shape, Index new_heads_number, const string& new_label)
{
    set(query_shape[0], query_shape[0], query_shape[1], new_heads_number, false, new_label);
}

MultiHeadAttention::MultiHeadAttention(const Shape& query_shape, const Shape& source_shape, Index new_heads_number, const string& new_label)
{
    if(query_shape[1] != source_shape[1])
        throw std::runtime_error("MultiHeadAttention Error: embedding dimension must be the same for query and source.");
    cross_attention = true;
    set(query_shape[0], source_shape[0], query_shape[1], new_heads_number, false, new_label);
}

void MultiHeadAttention::set(Index new_query_sequence_length, Index new_source_sequence_length, Index new_embedding_dimension,
                             Index new_heads_number, bool new_use_causal_mask, const string& new_label)
{
    name = "MultiHeadAttention";
    if(new_heads_number <= 0) throw std::runtime_error("MultiHeadAttention Error: Heads number must be greater than 0.");
    if(new_embedding_dimension % new_heads_number != 0)
        throw std::runtime_error("MultiHeadAttention Error: The embedding dimension must be divisible by the number of heads.");
    query_sequence_length = new_query_sequence_length;
    source_sequence_length = new_source_sequence_length;
    embedding_dimension = new_embedding_dimension;
    heads_number = new_heads_number;
    use_causal_mask = new_use_causal_mask;
    label = new_label;
    const Shape matrix = {embedding_dimension, embedding_dimension}, vector_shape = {embedding_dimension};
    query_weights_device.shape = key_weights_device.shape = value_weights_device.shape = projection_weights_device.shape = matrix;
    query_biases_device.shape = key_biases_device.shape = value_biases_device.shape = projection_biases_device.shape = vector_shape;
}

vector<TensorViewCuda*> MultiHeadAttention::get_parameter_views_device()
{
    return {&query_weights_device, &query_biases_device, &key_weights_device, &key_biases_device,
            &value_weights_device, &value_biases_device, &projection_weights_device, &projection_biases_device};
}

void MultiHeadAttention::set_parameters_random(vector<type>& host, Index offset, unsigned seed) const
{
    // U(-0.1, 0.1) for weights and biases (opennn/random_utilities.h:26 default range)
    std::mt19937 generator(seed);
    std::uniform_real_distribution<type> uniform(type(-0.1), type(0.1));
    const Index E = embedding_dimension;
    Index at = offset;
    for(int block = 0; block < 4; block++)
    {
        for(Index i = 0; i < E * E; i++) host[size_t(at + i)] = uniform(generator);
        at += padded(E * E);
        for(Index i = 0; i < E; i++) host[size_t(at + i)] = uniform(generator);
        at += padded(E);
    }
}

void MultiHeadAttentionForwardPropagationCuda::initialize()
{
    const MultiHeadAttention* mha = static_cast<const MultiHeadAttention*>(layer);
    outputs.shape = {batch_size, mha->get_query_sequence_length(), mha->get_embedding_dimension()};
    attention_state.shape = {Index(onn_mha_fwd_workspace_floats(batch_size, mha->get_query_sequence_length(),
                                                                mha->get_source_sequence_length(), mha->get_embedding_dimension(),
                                                                mha->get_heads_number()))};
}

vector<TensorViewCuda*> MultiHeadAttentionForwardPropagationCuda::get_workspace_views()
{
    vector<TensorViewCuda*> views = LayerForwardPropagationCuda::get_workspace_views();
    views.push_back(&attention_state);
    return views;
}

void MultiHeadAttentionBackPropagationCuda::initialize()
{
    const MultiHeadAttention* mha = static_cast<const MultiHeadAttention*>(layer);
    const Index E = mha->get_embedding_dimension();
    query_weight_gradients.shape = key_weight_gradients.shape = value_weight_gradients.shape = projection_weight_gradients.shape = {E, E};
    query_bias_gradients.shape = key_bias_gradients.shape = value_bias_gradients.shape = projection_bias_gradients.shape = {E};
    input_gradients.resize(mha->is_cross_attention() ? 2 : 1);
    input_gradients[0].shape = {batch_size, mha->get_query_sequence_length(), E};
    if(mha->is_cross_attention()) input_gradients[1].shape = {batch_size, mha->get_source_sequence_length(), E};
    scratch_floats = Index(onn_mha_bwd_workspace_floats(batch_size, mha->get_query_sequence_length(), mha->get_source_sequence_length(),
                                                        E, mha->get_heads_number()));
}

vector<TensorViewCuda*> MultiHeadAttentionBackPropagationCuda::get_gradient_views()
{
    // multihead_attention_layer.cpp:1215-1218: same order as the parameters
    return {&query_weight_gradients, &query_bias_gradients, &key_weight_gradients, &key_bias_gradients,
            &value_weight_gradients, &value_bias_gradients, &projection_weight_gradients, &projection_bias_gradients};
}

unique_ptr<LayerForwardPropagationCuda> MultiHeadAttention::create_forward_propagation() const { return std::make_unique<MultiHeadAttentionForwardPropagationCuda>(); }
unique_ptr<LayerBackPropagationCuda> MultiHeadAttention::create_back_propagation() const { return std::make_unique<MultiHeadAttentionBackPropagationCuda>(); }

void MultiHeadAttention::forward_propagate(unique_ptr<LayerForwardPropagationCuda>& forward, bool)
{
    MultiHeadAttentionForwardPropagationCuda* this_forward = static_cast<MultiHeadAttentionForwardPropagationCuda*>(forward.get());
    const type* query_input = forward->inputs[0].data;
    const type* source_input = forward->inputs.size() == 1 ? query_input : forward->inputs[1].data;   // multihead_attention_layer.cpp:192-194
    const onn_mha_params params = {query_weights_device.data, query_biases_device.data, key_weights_device.data, key_biases_device.data,
                                   value_weights_device.data, value_biases_device.data, projection_weights_device.data,
                                   projection_biases_device.data};
    check_onn(onn_mha_fwd(query_input, source_input, &params, this_forward->source_row_is_zero, forward->outputs.data,
                          forward->batch_size, query_sequence_length, source_sequence_length, embedding_dimension, heads_number,
                          use_causal_mask, this_forward->attention_state.data, 0, stream()),
              "MultiHeadAttention::forward_propagate");
}

void MultiHeadAttention::back_propagate(unique_ptr<LayerForwardPropagationCuda>& forward, unique_ptr<LayerBackPropagationCuda>& back) const
{
    MultiHeadAttentionForwardPropagationCuda* this_forward = static_cast<MultiHeadAttentionForwardPropagationCuda*>(forward.get());
    MultiHeadAttentionBackPropagationCuda* this_back = static_cast<MultiHeadAttentionBackPropagationCuda*>(back.get());
    const bool self_attention = forward->inputs.size() == 1;
    const type* query_input = forward->inputs[0].data;
    const type* source_input = self_attention ? query_input : forward->inputs[1].data;
    fold_extra_gradients(back->output_gradients, 1);

    const onn_mha_params params = {query_weights_device.data, query_biases_device.data, key_weights_device.data, key_biases_device.data,
                                   value_weights_device.data, value_biases_device.data, projection_weights_device.data,
                                   projection_biases_device.data};
    const onn_mha_grads grads = {this_back->query_weight_gradients.data, this_back->query_bias_gradients.data,
                                 this_back->key_weight_gradients.data, this_back->key_bias_gradients.data,
                                 this_back->value_weight_gradients.data, this_back->value_bias_gradients.data,
                                 this_back->projection_weight_gradients.data,
                                 this_back->projection_bias_gradient_is_ready ? nullptr : this_back->projection_bias_gradients.data};
    uint32_t flags = 0;
    if(!self_attention && back->accumulate_input_gradient.size() > 1 && back->accumulate_input_gradient[1]) flags |= ONN_ACCUMULATE;
    check_onn(onn_mha_bwd(query_input, source_input, &params, this_forward->attention_state.data, back->output_gradients[0].data, &grads,
                          back->input_gradients[0].data, self_attention ? nullptr : back->input_gradients[1].data,
                          forward->batch_size, query_sequence_length, source_sequence_length, embedding_dimension, heads_number,
                          use_causal_mask, this_back->scratch.data, flags, stream()),
              "MultiHeadAttention::back_propagate");
}


// ---------------------------------------------------------------------------------------
// Dense<3>
// ---------------------------------------------------------------------------------------

Dense3d::Dense3d(Index new_sequence_length, Index input_features, Index neurons, const string& activation, const string& new_label)
{
    name = "Dense3d";
    label = new_label;
    sequence_length = new_sequence_length;
    inputs_number = input_features;
    neurons_number = neurons;
    activation_function = activation;
    get_activation_code();                        // validates the name
    biases_device.shape = {neurons_number};
    weights_device.shape = {inputs_number, neurons_number};
}

int Dense3d::get_activation_code() const
{
    if(activation_function == "Linear") return ONN_ACT_LINEAR;
    if(activation_function == "RectifiedLinear") return ONN_ACT_RELU;
    if(activation_function == "Softmax") return ONN_ACT_SOFTMAX;
    if(activation_function == "Sigmoid" || activation_function == "Logistic") return ONN_ACT_SIGMOID;   // layer.h:129-136
    throw std::runtime_error("Unknown activation: " + activation_function);
}

void Dense3d::set_parameters_random(vector<type>& host, Index offset, unsigned seed) const
{
    // dense_layer.h:581-597: biases zero, weights U(-0.1, 0.1)
    std::mt19937 generator(seed);
    std::uniform_real_distribution<type> uniform(type(-0.1), type(0.1));
    for(Index i = 0; i < neurons_number; i++) host[size_t(offset + i)] = type(0);
    const Index weights_offset = offset + padded(neurons_number);
    for(Index i = 0; i < inputs_number * neurons_number; i++) host[size_t(weights_offset + i)] = uniform(generator);
}

void Dense3dForwardPropagationCuda::initialize()
{
    const Dense3d* dense = static_cast<const Dense3d*>(layer);
    outputs.shape = {batch_size, dense->get_sequence_length(), dense->get_neurons_number()};
    relu_bits.shape = {batch_size * dense->get_sequence_length(), Index(onn_relu_bits_words_per_row(dense->get_neurons_number()))};
}

vector<TensorViewCuda*> Dense3dForwardPropagationCuda::get_workspace_views()
{
    vector<TensorViewCuda*> views = LayerForwardPropagationCuda::get_workspace_views();
    if(wants_relu_bits) views.push_back(&relu_bits);
    return views;
}

void Dense3dBackPropagationCuda::initialize()
{
    const Dense3d* dense = static_cast<const Dense3d*>(layer);
    bias_gradients.shape = {dense->get_neurons_number()};
    weight_gradients.shape = {dense->get_input_features_number(), dense->get_neurons_number()};
    input_gradients.resize(1);
    input_gradients[0].shape = {batch_size, dense->get_sequence_length(), dense->get_input_features_number()};
}

unique_ptr<LayerForwardPropagationCuda> Dense3d::create_forward_propagation() const { return std::make_unique<Dense3dForwardPropagationCuda>(); }
unique_ptr<LayerBackPropagationCuda> Dense3d::create_back_propagation() const { return std::make_unique<Dense3dBackPropagationCuda>(); }

void Dense3d::forward_propagate(unique_ptr<LayerForwardPropagationCuda>& forward, bool is_training)
{
    Dense3dForwardPropagationCuda* this_forward = static_cast<Dense3dForwardPropagationCuda*>(forward.get());
    const Index rows = forward->batch_size * sequence_length;
    const uint32_t flags = (is_training && this_forward->defer_softmax) ? ONN_DEFER_SOFTMAX : 0;
    uint32_t* relu_bits = (is_training && this_forward->wants_relu_bits) ? reinterpret_cast<uint32_t*>(this_forward->relu_bits.data) : nullptr;
    check_onn(onn_dense_fwd(forward->inputs[0].data, weights_device.data, biases_device.data, forward->outputs.data, relu_bits,
                            rows, inputs_number, neurons_number, get_activation_code(), flags, stream()),
              "Dense3d::forward_propagate");
}

void Dense3d::back_propagate(unique_ptr<LayerForwardPropagationCuda>& forward, unique_ptr<LayerBackPropagationCuda>& back) const
{
    Dense3dBackPropagationCuda* this_back = static_cast<Dense3dBackPropagationCuda*>(back.get());
    const Index rows = forward->batch_size * sequence_length;
    fold_extra_gradients(back->output_gradients, 1);
    const uint32_t flags = this_back->delta_is_ready ? ONN_DELTA_READY : 0;
    check_onn(onn_dense_bwd(forward->inputs[0].data, weights_device.data, forward->outputs.data, back->output_gradients[0].data,
                            this_back->weight_gradients.data, this_back->bias_gradient_is_ready ? nullptr : this_back->bias_gradients.data,
                            this_back->skip_input_gradient ? nullptr : back->input_gradients[0].data, this_back->input_relu_mask,
                            this_back->input_relu_bits, this_back->input_bias_gradients,
                            rows, inputs_number, neurons_number, get_activation_code(), flags, stream()),
              "Dense3d::back_propagate");
}


// ---------------------------------------------------------------------------------------
// Normalization3d and Addition<3>
// ---------------------------------------------------------------------------------------

unique_ptr<Dense3d> Dense3d::make_rank2(Index input_features, Index neurons, const string& activation, const string& new_label)
{
    unique_ptr<Dense3d> layer = std::make_unique<Dense3d>(1, input_features, neurons, activation, new_label);
    layer->name = "Dense2d";
    return layer;
}


// ---------------------------------------------------------------------------------------
// Pooling3d
// ---------------------------------------------------------------------------------------

Pooling3d::Pooling3d(const Shape& input_shape, PoolingMethod method, const string& new_label)
{
    name = "Pooling3d";
    label = new_label;
    sequence_length = input_shape[0];
    features = input_shape[1];
    pooling_method = method;
}

void Pooling3dForwardPropagationCuda::initialize()
{
    const Shape input = layer->get_input_shape();
    outputs.shape = {batch_size, input[1]};
    maximal_indices.shape = {batch_size, input[1]};
    row_is_valid.shape = {(batch_size * input[0] + 3) / 4};
    valid_count.shape = {batch_size};
}

vector<TensorViewCuda*> Pooling3dForwardPropagationCuda::get_workspace_views()
{
    vector<TensorViewCuda*> views = LayerForwardPropagationCuda::get_workspace_views();
    views.push_back(&maximal_indices);
    views.push_back(&row_is_valid);
    views.push_back(&valid_count);
    return views;
}

void Pooling3dBackPropagationCuda::initialize()
{
    const Shape input = layer->get_input_shape();
    input_gradients.resize(1);
    input_gradients[0].shape = {batch_size, input[0], input[1]};
}

unique_ptr<LayerForwardPropagationCuda> Pooling3d::create_forward_propagation() const { return std::make_unique<Pooling3dForwardPropagationCuda>(); }
unique_ptr<LayerBackPropagationCuda> Pooling3d::create_back_propagation() const { return std::make_unique<Pooling3dBackPropagationCuda>(); }

void Pooling3d::forward_propagate(unique_ptr<LayerForwardPropagationCuda>& forward, bool)
{
    Pooling3dForwardPropagationCuda* state = static_cast<Pooling3dForwardPropagationCuda*>(forward.get());
    check_onn(onn_pooling3d_fwd(forward->inputs[0].data, forward->outputs.data, reinterpret_cast<int32_t*>(state->maximal_indices.data),
                                reinterpret_cast<uint8_t*>(state->row_is_valid.data), reinterpret_cast<int32_t*>(state->valid_count.data),
                                forward->batch_size, sequence_length, features,
                                pooling_method == PoolingMethod::MaxPooling ? ONN_POOL_MAX : ONN_POOL_AVERAGE, stream()),
              "Pooling3d::forward_propagate");
}

void Pooling3d::back_propagate(unique_ptr<LayerForwardPropagationCuda>& forward, unique_ptr<LayerBackPropagationCuda>& back) const
{
    Pooling3dForwardPropagationCuda* state = static_cast<Pooling3dForwardPropagationCuda*>(forward.get());
    fold_extra_gradients(back->output_gradients, 1);
    check_onn(onn_pooling3d_bwd(back->output_gradients[0].data, reinterpret_cast<const int32_t*>(state->maximal_indices.data),
                                reinterpret_cast<const uint8_t*>(state->row_is_valid.data), reinterpret_cast<const int32_t*>(state->valid_count.data),
                                back->input_gradients[0].data, forward->batch_size, sequence_length, features,
                                pooling_method == PoolingMethod::MaxPooling ? ONN_POOL_MAX : ONN_POOL_AVERAGE, stream()),
              "Pooling3d::back_propagate");
}


Normalization3d::Normalization3d(const Shape& input_shape, const string& new_label)
{
    name = "Normalization3d";
    label = new_label;
    sequence_length = input_shape[0];
    embedding_dimension = input_shape[1];
    gammas_device.shape = {embedding_dimension};
    betas_device.shape = {embedding_dimension};
}

void Normalization3d::set_parameters_random(vector<type>& host, Index offset, unsigned) const
{
    // normalization_layer_3d.cpp:72-79: gammas one, betas zero
    for(Index i = 0; i < embedding_dimension; i++) host[size_t(offset + i)] = type(1);
    for(Index i = 0; i < embedding_dimension; i++) host[size_t(offset + padded(embedding_dimension) + i)] = type(0);
}

void Normalization3dForwardPropagationCuda::initialize()
{
    const Normalization3d* norm = static_cast<const Normalization3d*>(layer);
    outputs.shape = {batch_size, norm->get_sequence_length(), norm->get_embedding_dimension()};
    means.shape = {batch_size, norm->get_sequence_length()};
    inverse_standard_deviations.shape = {batch_size, norm->get_sequence_length()};
    outputs_row_is_zero.shape = {(batch_size * norm->get_sequence_length() + 3) / 4};
}

vector<TensorViewCuda*> Normalization3dForwardPropagationCuda::get_workspace_views()
{
    vector<TensorViewCuda*> views = LayerForwardPropagationCuda::get_workspace_views();
    views.push_back(&means);
    views.push_back(&inverse_standard_deviations);
    return views;
}

void Normalization3dBackPropagationCuda::initialize()
{
    const Normalization3d* norm = static_cast<const Normalization3d*>(layer);
    gamma_gradients.shape = {norm->get_embedding_dimension()};
    beta_gradients.shape = {norm->get_embedding_dimension()};
    input_gradients.resize(1);
    input_gradients[0].shape = {batch_size, norm->get_sequence_length(), norm->get_embedding_dimension()};
    partial_sums.shape = {Index(onn_layernorm_bwd_workspace_floats(batch_size * norm->get_sequence_length(), norm->get_embedding_dimension()))};
}

vector<TensorViewCuda*> Normalization3dBackPropagationCuda::get_workspace_views()
{
    vector<TensorViewCuda*> views = LayerBackPropagationCuda::get_workspace_views();
    views.push_back(&partial_sums);
    return views;
}

unique_ptr<LayerForwardPropagationCuda> Normalization3d::create_forward_propagation() const { return std::make_unique<Normalization3dForwardPropagationCuda>(); }
unique_ptr<LayerBackPropagationCuda> Normalization3d::create_back_propagation() const { return std::make_unique<Normalization3dBackPropagationCuda>(); }

void Normalization3d::forward_propagate(unique_ptr<LayerForwardPropagationCuda>& forward, bool)
{
    Normalization3dForwardPropagationCuda* this_forward = static_cast<Normalization3dForwardPropagationCuda*>(forward.get());
    const Index rows = forward->batch_size * sequence_length;
    const bool fused_addition = this_forward->addend_a != nullptr;
    check_onn(onn_layernorm_fwd(fused_addition ? this_forward->addend_a : forward->inputs[0].data,
                                fused_addition ? this_forward->addend_b : nullptr,
                                gammas_device.data, betas_device.data, forward->outputs.data,
                                fused_addition ? this_forward->sum_output : nullptr,
                                this_forward->means.data, this_forward->inverse_standard_deviations.data, row_flags_of(*forward),
                                rows, embedding_dimension, EPSILON, 0, stream()),
              "Normalization3d::forward_propagate");
}

void Normalization3d::back_propagate(unique_ptr<LayerForwardPropagationCuda>& forward, unique_ptr<LayerBackPropagationCuda>& back) const
{
    Normalization3dForwardPropagationCuda* this_forward = static_cast<Normalization3dForwardPropagationCuda*>(forward.get());
    Normalization3dBackPropagationCuda* this_back = static_cast<Normalization3dBackPropagationCuda*>(back.get());
    const Index rows = forward->batch_size * sequence_length;
    const vector<TensorViewCuda>& gradients = back->output_gradients;
    fold_extra_gradients(gradients, 3);
    check_onn(onn_layernorm_bwd(gradients[0].data, gradients.size() > 1 ? gradients[1].data : nullptr,
                                gradients.size() > 2 ? gradients[2].data : nullptr, forward->inputs[0].data,
                                this_forward->means.data, this_forward->inverse_standard_deviations.data, gammas_device.data,
                                back->input_gradients[0].data, this_back->gamma_gradients.data, this_back->beta_gradients.data,
                                this_back->input_bias_gradients,
                                rows, embedding_dimension, this_back->partial_sums.data, ONN_ACCUMULATE, stream()),
              "Normalization3d::back_propagate");
}

Addition3d::Addition3d(const Shape& input_shape, const string& new_label)
{
    name = "Addition3d";
    label = new_label;
    sequence_length = input_shape[0];
    embedding_dimension = input_shape[1];
}

void Addition3dForwardPropagationCuda::initialize()
{
    outputs.shape = {batch_size, layer->get_output_shape()[0], layer->get_output_shape()[1]};
}

void Addition3dBackPropagationCuda::initialize()
{
    input_gradients.resize(2);
    input_gradients[0].shape = input_gradients[1].shape = {batch_size, layer->get_output_shape()[0], layer->get_output_shape()[1]};
}

unique_ptr<LayerForwardPropagationCuda> Addition3d::create_forward_propagation() const { return std::make_unique<Addition3dForwardPropagationCuda>(); }
unique_ptr<LayerBackPropagationCuda> Addition3d::create_back_propagation() const { return std::make_unique<Addition3dBackPropagationCuda>(); }

void Addition3d::forward_propagate(unique_ptr<LayerForwardPropagationCuda>& forward, bool)
{
    if(forward->fused_into_consumer) return;      // the following Normalization3d computes and stores the sum
    check_onn(onn_add(forward->inputs[0].data, forward->inputs[1].data, forward->outputs.data, forward->outputs.size(), 0, stream()),
              "Addition3d::forward_propagate");
}

void Addition3d::back_propagate(unique_ptr<LayerForwardPropagationCuda>&, unique_ptr<LayerBackPropagationCuda>& back) const
{
    if(back->fused_into_consumer) return;         // both input gradients alias the consumer's input gradient
    // addition_layer.h:148-168: the output gradient goes to both inputs
    fold_extra_gradients(back->output_gradients, 1);
    const size_t bytes = size_t(back->output_gradients[0].size()) * sizeof(type);
    for(int port = 0; port < 2; port++)
        check_cuda(cudaMemcpyAsync(back->input_gradients[port].data, back->output_gradients[0].data, bytes, cudaMemcpyDeviceToDevice,
                                   Device::instance().get_compute_stream()), "Addition3d::back_propagate");
}

}  // namespace opennn_b200
