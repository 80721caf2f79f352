// Test infrastructure: drives the UNMODIFIED OpenNN CPU (Eigen) path on seeded inputs read
// from raw little-endian fp32 files, and dumps outputs / loss / gradients / updated
// parameters.  It is the checker for the CUDA path and the timed CPU baseline; nothing in
// the product links or calls it.
//
//   onn_ref_harness <dir>
//
// <dir>/spec.txt holds "key=value" lines; every tensor is <dir>/<name>.bin (fp32, row-major).
// Modes (spec key "mode"):
//   layer        one layer driven with the fixture pattern of the reference's own layer
//                tests (tests/multihead_attention_layer_test.cpp:66-92, 161-201):
//                kind = mha | embedding | layernorm | dense
//   ce3d         CrossEntropyError3d on given probabilities
//                (cross_entropy_error_3d.cpp:78-136, 154-247)
//   transformer  Transformer (standard_networks.cpp:638-907) + CrossEntropyError3d + Adam,
//                the loop body of adaptive_moment_estimation.cpp:249-284
//   decoder      decoder-only stack assembled with add_layer the way Transformer::set
//                assembles its decoder, minus cross-attention
//   transformer_cuda / decoder_cuda   (only in the binary built with the reference's CUDA path,
//                `make -C oracle cuda`): the same networks through the reference's OWN GPU path,
//                the loop body of AdaptiveMomentEstimation::train_cuda
//                (adaptive_moment_estimation.cpp:697-721): cuBLAS SGEMM + cuDNN + opennn/kernel.cu.
//                Timed per step with a device synchronisation on both sides; it is the
//                "existing GPU implementation" the new path is compared with, nothing more.
//
// Token ids and targets are floats holding integers, as in the reference (dataset.h:525-558).

#include "opennn.h"

#include <chrono>

using namespace opennn;

namespace
{

map<string, string> spec;
string dir_path;

string spec_string(const string& key, const string& fallback = "")
{
    const auto it = spec.find(key);
    return it == spec.end() ? fallback : it->second;
}

Index spec_index(const string& key, Index fallback = 0)
{
    const auto it = spec.find(key);
    return it == spec.end() ? fallback : Index(stoll(it->second));
}

double spec_double(const string& key, double fallback = 0)
{
    const auto it = spec.find(key);
    return it == spec.end() ? fallback : stod(it->second);
}

void read_spec()
{
    ifstream file(dir_path + "/spec.txt");
    if(!file) throw runtime_error("cannot open spec.txt in " + dir_path);
    string line;
    while(getline(file, line))
    {
        const size_t eq = line.find('=');
        if(eq == string::npos) continue;
        spec[line.substr(0, eq)] = line.substr(eq + 1);
    }
}

vector<type> read_bin(const string& name, Index expected = -1)
{
    ifstream file(dir_path + "/" + name + ".bin", ios::binary | ios::ate);
    if(!file) throw runtime_error("cannot open " + name + ".bin");
    const Index bytes = Index(file.tellg());
    file.seekg(0);
    vector<type> data(bytes / sizeof(type));
    file.read(reinterpret_cast<char*>(data.data()), bytes);
    if(expected >= 0 && Index(data.size()) != expected)
        throw runtime_error(name + ".bin: expected " + to_string(expected) + " floats, got " + to_string(data.size()));
    return data;
}

void write_bin(const string& name, const type* data, Index count)
{
    ofstream file(dir_path + "/" + name + ".bin", ios::binary);
    file.write(reinterpret_cast<const char*>(data), count * sizeof(type));
}

double now_seconds()
{
    return chrono::duration<double>(chrono::steady_clock::now().time_since_epoch()).count();
}


// One layer, driven directly through the Layer virtuals.

unique_ptr<Layer> make_layer(const string& kind, Index& inputs_count, vector<Shape>& input_shapes, Index batch)
{
    const Index S = spec_index("S");
    const Index E = spec_index("E");

    if(kind == "mha")
    {
        const Index Sk = spec_index("Sk", S);
        const Index H = spec_index("H");
        const bool cross = spec_index("cross") != 0;
        const bool causal = spec_index("causal") != 0;

        unique_ptr<MultiHeadAttention> layer = cross
            ? make_unique<MultiHeadAttention>(Shape{S, E}, Shape{Sk, E}, H)
            : make_unique<MultiHeadAttention>(Shape{S, E}, H);
        layer->set(S, Sk, E, H, causal);

        inputs_count = cross ? 2 : 1;
        input_shapes = {Shape{batch, S, E}};
        if(cross) input_shapes.push_back(Shape{batch, Sk, E});
        return layer;
    }

    if(kind == "embedding")
    {
        const Index V = spec_index("V");
        unique_ptr<Embedding> layer = make_unique<Embedding>(Shape{V, S}, E);
        layer->set_scale_embedding(spec_index("scale", 1) != 0);
        layer->set_add_positional_encoding(spec_index("add_pe", 1) != 0);
        inputs_count = 1;
        input_shapes = {Shape{batch, S}};
        return layer;
    }

    if(kind == "layernorm")
    {
        inputs_count = 1;
        input_shapes = {Shape{batch, S, E}};
        return make_unique<Normalization3d>(Shape{S, E});
    }

    if(kind == "dense")
    {
        const Index F = spec_index("F");
        inputs_count = 1;
        input_shapes = {Shape{batch, S, E}};
        return make_unique<opennn::Dense<3>>(S, E, F, spec_string("activation", "Linear"), "dense");
    }

    if(kind == "pooling3d")
    {
        inputs_count = 1;
        input_shapes = {Shape{batch, S, E}};
        const Pooling3d::PoolingMethod method = spec_string("method", "MaxPooling") == "MaxPooling"
            ? Pooling3d::PoolingMethod::MaxPooling : Pooling3d::PoolingMethod::AveragePooling;
        return make_unique<Pooling3d>(Shape{S, E}, method);
    }

    throw runtime_error("unknown layer kind " + kind);
}


void run_layer()
{
    const string kind = spec_string("kind");
    const Index B = spec_index("B");

    Index inputs_count = 0;
    vector<Shape> input_shapes;
    unique_ptr<Layer> layer = make_layer(kind, inputs_count, input_shapes, B);

    vector<TensorView*> parameter_views = layer->get_parameter_views();
    VectorR parameters(get_size(parameter_views));
    parameters.setZero();
    if(parameters.size() > 0)                                   // Pooling3d has none
    {
        link(parameters.data(), parameter_views);
        const vector<type> parameters_in = read_bin("params", parameters.size());
        memcpy(parameters.data(), parameters_in.data(), parameters_in.size() * sizeof(type));
    }

    vector<VectorR> inputs(inputs_count);
    for(Index i = 0; i < inputs_count; i++)
    {
        const vector<type> data = read_bin("x" + to_string(i), input_shapes[i].count());
        inputs[i].resize(data.size());
        memcpy(inputs[i].data(), data.data(), data.size() * sizeof(type));
    }

    unique_ptr<LayerForwardPropagation> forward = Registry<LayerForwardPropagation>::instance().create(layer->get_name());
    forward->set(B, layer.get());

    VectorR forward_workspace(get_size(forward->get_workspace_views()));
    forward_workspace.setZero();
    link(forward_workspace.data(), forward->get_workspace_views());

    forward->inputs.resize(inputs_count);
    for(Index i = 0; i < inputs_count; i++)
        forward->inputs[i] = TensorView(inputs[i].data(), input_shapes[i]);

    layer->forward_propagate(forward, true);

    const TensorView outputs = forward->get_outputs();
    write_bin("y", outputs.data, outputs.size());

    if(kind == "mha")
    {
        MultiHeadAttentionForwardPropagation* mha = static_cast<MultiHeadAttentionForwardPropagation*>(forward.get());
        write_bin("attention_weights", mha->attention_weights.data(), mha->attention_weights.size());
    }

    if(spec_index("backward", 1) == 0) return;

    unique_ptr<LayerBackPropagation> back = Registry<LayerBackPropagation>::instance().create(layer->get_name());
    back->set(B, layer.get());

    vector<TensorView*> gradient_views = back->get_gradient_views();
    VectorR gradients(get_size(gradient_views));
    gradients.setZero();
    if(gradients.size() > 0) link(gradients.data(), gradient_views);

    vector<TensorView*> back_workspace_views = back->get_workspace_views();
    VectorR back_workspace(get_size(back_workspace_views));
    back_workspace.setZero();
    if(back_workspace.size() > 0)
        link(back_workspace.data(), back_workspace_views);

    vector<type> deltas = read_bin("delta", outputs.size());
    back->output_gradients = { TensorView(deltas.data(), outputs.shape) };

    layer->back_propagate(forward, back);

    write_bin("grads", gradients.data(), gradients.size());

    for(size_t i = 0; i < back->input_gradients.size(); i++)
        if(back->input_gradients[i].data && kind != "embedding")
            write_bin("dx" + to_string(i), back->input_gradients[i].data, back->input_gradients[i].size());
}


// The loss alone, on probabilities handed in as the "outputs" of a one-layer network.

void run_ce3d()
{
    const Index B = spec_index("B");
    const Index S = spec_index("S");
    const Index V = spec_index("V");

    // A Dense<3> softmax layer gives the loss a network whose last outputs are [B,S,V];
    // its forward pass is not run: the probabilities are written over its output buffer.
    NeuralNetwork network;
    network.add_layer(unique_ptr<Layer>(new opennn::Dense<3>(Shape{S, 2}, Shape{V}, "Softmax")));
    network.set_parameters_random();

    CrossEntropyError3d loss(&network, nullptr);
    loss.set_regularization_method("None");

    Batch batch;
    batch.samples_number = B;
    batch.input_shape = {B, S, 2};
    batch.input_vector.resize(B * S * 2);
    batch.input_vector.setZero();
    batch.target_shape = {B, S};
    const vector<type> targets = read_bin("targets", B * S);
    batch.target_vector.resize(B * S);
    memcpy(batch.target_vector.data(), targets.data(), targets.size() * sizeof(type));

    ForwardPropagation forward(B, &network);
    network.forward_propagate(batch.get_inputs(), forward, true);

    const vector<type> probabilities = read_bin("p", B * S * V);
    TensorView outputs = forward.get_last_trainable_layer_outputs();
    memcpy(outputs.data, probabilities.data(), probabilities.size() * sizeof(type));

    BackPropagation back(B, &loss);
    loss.calculate_error(batch, forward, back);
    loss.calculate_output_gradients(batch, forward, back);

    const type scalars[2] = { back.error, back.accuracy(0) };
    write_bin("loss", scalars, 2);
    const TensorView output_gradients = back.get_output_gradients();
    write_bin("dlogits", output_gradients.data, output_gradients.size());
}


// Whole network: forward, loss, backward, Adam.

void build_decoder_only(NeuralNetwork& network, Index S, Index V, Index E, Index H, Index F, Index L)
{
    network.reference_all_layers();

    unique_ptr<Embedding> embedding = make_unique<Embedding>(Shape{V, S}, E, "decoder_embedding");
    embedding->set_scale_embedding(true);
    embedding->set_add_positional_encoding(true);
    network.add_layer(move(embedding), {-1});

    Index current = network.get_layers_number() - 1;

    for(Index i = 0; i < L; i++)
    {
        const string suffix = "_" + to_string(i + 1);

        unique_ptr<MultiHeadAttention> attention = make_unique<MultiHeadAttention>(Shape{S, E}, H, "decoder_self_attention" + suffix);
        attention->set(S, S, E, H, true, "decoder_self_attention" + suffix);
        network.add_layer(move(attention), {current});
        const Index attention_index = network.get_layers_number() - 1;

        network.add_layer(make_unique<Addition<3>>(Shape{S, E}, "decoder_self_attention_addition" + suffix), {current, attention_index});
        network.add_layer(make_unique<Normalization3d>(Shape{S, E}, "decoder_self_attention_normalization" + suffix));
        const Index norm_index = network.get_layers_number() - 1;

        network.add_layer(make_unique<opennn::Dense<3>>(S, E, F, "RectifiedLinear", "decoder_internal_dense" + suffix));
        network.add_layer(make_unique<opennn::Dense<3>>(S, F, E, "Linear", "decoder_external_dense" + suffix));
        const Index dense_index = network.get_layers_number() - 1;

        network.add_layer(make_unique<Addition<3>>(Shape{S, E}, "decoder_dense_addition" + suffix), {norm_index, dense_index});
        network.add_layer(make_unique<Normalization3d>(Shape{S, E}, "decoder_dense_normalization" + suffix));
        current = network.get_layers_number() - 1;
    }

    network.add_layer(make_unique<opennn::Dense<3>>(S, E, V, "Softmax", "output_projection"));
    network.compile();
    network.set_parameters_random();
}


void run_network(bool decoder_only)
{
    const Index B = spec_index("B");
    const Index S_in = spec_index("S_in");
    const Index S_dec = spec_index("S_dec");
    const Index V_in = spec_index("V_in");
    const Index V_out = spec_index("V_out");
    const Index E = spec_index("E");
    const Index H = spec_index("H");
    const Index F = spec_index("F");
    const Index L = spec_index("L");
    const Index steps = spec_index("steps", 1);
    const bool dump_layers = spec_index("dump_layers") != 0;
    const bool dump = spec_index("dump", 1) != 0;
    const bool random_parameters = spec_index("random_parameters") != 0;

    unique_ptr<NeuralNetwork> network;
    if(decoder_only)
    {
        network = make_unique<NeuralNetwork>();
        build_decoder_only(*network, S_dec, V_out, E, H, F, L);
    }
    else
        network = make_unique<Transformer>(S_in, S_dec, V_in, V_out, E, H, F, L);

    VectorR& parameters = network->get_parameters();

    {
        const type count[2] = { type(parameters.size()), type(network->get_layers_number()) };
        write_bin("param_count", count, 2);
        ofstream names(dir_path + "/layers.txt");
        for(const unique_ptr<Layer>& layer : network->get_layers())
            names << layer->get_name() << " " << layer->get_label() << " " << get_size(layer->get_parameter_views()) << "\n";
    }

    if(spec_index("structure_only") != 0) return;

    if(!random_parameters)
    {
        const vector<type> parameters_in = read_bin("params", parameters.size());
        memcpy(parameters.data(), parameters_in.data(), parameters_in.size() * sizeof(type));
    }

    CrossEntropyError3d loss(network.get(), nullptr);
    loss.set_regularization_method("None");

    Batch batch;
    batch.samples_number = B;

    if(!decoder_only)
    {
        const vector<type> encoder_ids = read_bin("enc_ids", B * S_in);
        batch.input_shape = {B, S_in};
        batch.input_vector.resize(B * S_in);
        memcpy(batch.input_vector.data(), encoder_ids.data(), encoder_ids.size() * sizeof(type));

        const vector<type> decoder_ids = read_bin("dec_ids", B * S_dec);
        batch.decoder_shape = {B, S_dec};
        batch.decoder_vector.resize(B * S_dec);
        memcpy(batch.decoder_vector.data(), decoder_ids.data(), decoder_ids.size() * sizeof(type));
    }
    else
    {
        const vector<type> decoder_ids = read_bin("dec_ids", B * S_dec);
        batch.input_shape = {B, S_dec};
        batch.input_vector.resize(B * S_dec);
        memcpy(batch.input_vector.data(), decoder_ids.data(), decoder_ids.size() * sizeof(type));
    }

    const vector<type> targets = read_bin("targets", B * S_dec);
    batch.target_shape = {B, S_dec};
    batch.target_vector.resize(B * S_dec);
    memcpy(batch.target_vector.data(), targets.data(), targets.size() * sizeof(type));

    ForwardPropagation forward(B, network.get());
    BackPropagation back(B, &loss);

    AdaptiveMomentEstimation adam(&loss);
    adam.set_learning_rate(type(spec_double("lr", 1e-3)));
    AdaptiveMomentEstimationData optimization_data(&adam);
    optimization_data.iteration = 1;

    vector<type> history;
    vector<double> step_seconds;

    for(Index step = 0; step < steps; step++)
    {
        const double start = now_seconds();

        back.neural_network.gradient.setZero();
        network->forward_propagate(batch.get_inputs(), forward, true);
        loss.back_propagate(batch, forward, back);

        if(step == 0 && dump)
        {
            write_bin("grad_step0", back.neural_network.gradient.data(), back.neural_network.gradient.size());

            if(dump_layers)
                for(size_t i = 0; i < forward.layers.size(); i++)
                {
                    const TensorView outputs = forward.layers[i]->get_outputs();
                    write_bin("layer_out_" + to_string(i), outputs.data, outputs.size());
                }
        }

        adam.update_parameters(back, optimization_data);

        step_seconds.push_back(now_seconds() - start);
        history.push_back(back.error);
        history.push_back(back.accuracy(0));
    }

    write_bin("loss", history.data(), history.size());
    if(dump)
        write_bin("params_out", parameters.data(), parameters.size());

    ofstream timing(dir_path + "/timing.txt");
    for(const double seconds : step_seconds) timing << seconds << "\n";
}



#ifdef OPENNN_CUDA

// The reference's own CUDA training step on a batch made by hand (BatchCuda needs a Dataset only to size itself:
// dataset.cpp:4397-4460; its members are public).
void run_network_cuda(bool decoder_only)
{
    const Index B = spec_index("B");
    const Index S_in = spec_index("S_in");
    const Index S_dec = spec_index("S_dec");
    const Index V_in = spec_index("V_in");
    const Index V_out = spec_index("V_out");
    const Index E = spec_index("E");
    const Index H = spec_index("H");
    const Index F = spec_index("F");
    const Index L = spec_index("L");
    const Index steps = spec_index("steps", 1);

    unique_ptr<NeuralNetwork> network;
    if(decoder_only)
    {
        network = make_unique<NeuralNetwork>();
        build_decoder_only(*network, S_dec, V_out, E, H, F, L);
    }
    else
        network = make_unique<Transformer>(S_in, S_dec, V_in, V_out, E, H, F, L);

    VectorR& parameters = network->get_parameters();
    if(spec_index("random_parameters") == 0)
    {
        const vector<type> parameters_in = read_bin("params", parameters.size());
        memcpy(parameters.data(), parameters_in.data(), parameters_in.size() * sizeof(type));
    }

    CrossEntropyError3d loss(network.get(), nullptr);
    loss.set_regularization_method("None");

    BatchCuda batch;
    batch.samples_number = B;
    const vector<type> targets = read_bin("targets", B * S_dec);
    const vector<type> decoder_ids = read_bin("dec_ids", B * S_dec);
    if(!decoder_only)
    {
        const vector<type> encoder_ids = read_bin("enc_ids", B * S_in);
        batch.input_shape = {B, S_in};
        batch.num_input_features = S_in;
        batch.inputs_device.resize({B, S_in});
        CHECK_CUDA(cudaMemcpy(batch.inputs_device.data, encoder_ids.data(), encoder_ids.size() * sizeof(type), cudaMemcpyHostToDevice));
        batch.decoder_shape = {B, S_dec};
        batch.num_decoder_features = S_dec;
        batch.decoder_device.resize({B, S_dec});
        CHECK_CUDA(cudaMemcpy(batch.decoder_device.data, decoder_ids.data(), decoder_ids.size() * sizeof(type), cudaMemcpyHostToDevice));
    }
    else
    {
        batch.input_shape = {B, S_dec};
        batch.num_input_features = S_dec;
        batch.inputs_device.resize({B, S_dec});
        CHECK_CUDA(cudaMemcpy(batch.inputs_device.data, decoder_ids.data(), decoder_ids.size() * sizeof(type), cudaMemcpyHostToDevice));
    }
    batch.target_shape = {B, S_dec};
    batch.num_target_features = S_dec;
    batch.targets_device.resize({B, S_dec});
    CHECK_CUDA(cudaMemcpy(batch.targets_device.data, targets.data(), targets.size() * sizeof(type), cudaMemcpyHostToDevice));

    ForwardPropagationCuda forward(B, network.get());
    network->copy_parameters_device();
    BackPropagationCuda back(B, &loss);

    AdaptiveMomentEstimation adam(&loss);
    adam.set_learning_rate(type(spec_double("lr", 1e-3)));
    ADAMOptimizationDataCuda optimization_data(&adam);
    optimization_data.iteration = 1;

    vector<type> history;
    vector<double> step_seconds;
    for(Index step = 0; step < steps; step++)
    {
        CHECK_CUDA(cudaDeviceSynchronize());
        const double start = now_seconds();

        back.neural_network.gradients.fill(0.0f);
        network->forward_propagate(batch.get_inputs_device(), forward, true);
        loss.back_propagate(batch, forward, back);
        adam.update_parameters(back, optimization_data);

        CHECK_CUDA(cudaDeviceSynchronize());
        step_seconds.push_back(now_seconds() - start);
        history.push_back(back.error);
        history.push_back(back.accuracy(0));
    }

    write_bin("loss", history.data(), history.size());
    ofstream timing(dir_path + "/timing.txt");
    for(const double seconds : step_seconds) timing << seconds << "\n";
}

#endif


// Text classifier (Embedding -> MultiHeadAttention -> Pooling3d -> Dense<2>... -> Softmax) with CrossEntropyError2d.

void run_classifier()
{
    const Index B = spec_index("B");
    const Index S = spec_index("S");
    const Index V = spec_index("V");
    const Index E = spec_index("E");
    const Index H = spec_index("H");
    const Index hidden = spec_index("hidden");
    const Index classes = spec_index("classes");
    const Index steps = spec_index("steps", 1);

    Shape complexity;
    if(hidden > 0) complexity.push_back(hidden);
    TextClassificationNetwork network(Shape{V, S, E, H}, complexity, Shape{classes});

    VectorR& parameters = network.get_parameters();
    {
        const type count[2] = { type(parameters.size()), type(network.get_layers_number()) };
        write_bin("param_count", count, 2);
        ofstream names(dir_path + "/layers.txt");
        for(const unique_ptr<Layer>& layer : network.get_layers())
            names << layer->get_name() << " " << layer->get_label() << " " << get_size(layer->get_parameter_views()) << "\n";
    }
    if(spec_index("structure_only") != 0) return;

    const vector<type> parameters_in = read_bin("params", parameters.size());
    memcpy(parameters.data(), parameters_in.data(), parameters_in.size() * sizeof(type));

    CrossEntropyError2d loss(&network, nullptr);
    loss.set_regularization_method("None");

    Batch batch;
    batch.samples_number = B;
    const vector<type> ids = read_bin("ids", B * S);
    batch.input_shape = {B, S};
    batch.input_vector.resize(B * S);
    memcpy(batch.input_vector.data(), ids.data(), ids.size() * sizeof(type));
    const vector<type> targets = read_bin("targets", B * classes);
    batch.target_shape = {B, classes};
    batch.target_vector.resize(B * classes);
    memcpy(batch.target_vector.data(), targets.data(), targets.size() * sizeof(type));

    ForwardPropagation forward(B, &network);
    BackPropagation back(B, &loss);
    AdaptiveMomentEstimation adam(&loss);
    adam.set_learning_rate(type(spec_double("lr", 1e-3)));
    AdaptiveMomentEstimationData optimization_data(&adam);
    optimization_data.iteration = 1;

    vector<type> history;
    for(Index step = 0; step < steps; step++)
    {
        back.neural_network.gradient.setZero();
        network.forward_propagate(batch.get_inputs(), forward, true);
        loss.back_propagate(batch, forward, back);
        if(step == 0)
        {
            write_bin("grad_step0", back.neural_network.gradient.data(), back.neural_network.gradient.size());
            const TensorView outputs = forward.get_outputs();
            write_bin("probabilities", outputs.data, outputs.size());
        }
        adam.update_parameters(back, optimization_data);
        history.push_back(back.error);
    }
    write_bin("loss", history.data(), history.size());
    write_bin("params_out", parameters.data(), parameters.size());
}

}


int main(int argc, char** argv)
{
    if(argc < 2)
    {
        cerr << "usage: onn_ref_harness <dir>" << endl;
        return 2;
    }

    try
    {
        dir_path = argv[1];
        read_spec();

        const int threads = int(spec_index("threads", omp_get_max_threads()));
        omp_set_num_threads(threads);
        Device::instance().set_threads_number(threads);

        const string mode = spec_string("mode");

        if(mode == "layer") run_layer();
        else if(mode == "ce3d") run_ce3d();
        else if(mode == "transformer") run_network(false);
        else if(mode == "decoder") run_network(true);
#ifdef OPENNN_CUDA
        else if(mode == "transformer_cuda") run_network_cuda(false);
        else if(mode == "decoder_cuda") run_network_cuda(true);
#endif
        else if(mode == "classifier") run_classifier();
        else throw runtime_error("unknown mode " + mode);
    }
    catch(const exception& e)
    {
        cerr << "onn_ref_harness: " << e.what() << endl;
        return 1;
    }

    return 0;
}
