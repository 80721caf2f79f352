// C driver ABI for the text-classification network (include/onn_b200_host.h, onn_classifier_*): builds
// TextClassificationNetwork (opennn/standard_networks.cpp:575-615) with CrossEntropyError2d and Adam and runs the body
// of the training loop (opennn/adaptive_moment_estimation.cpp:697-718) one optimiser step at a time on one GPU.
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "../../include/onn_b200_host.h"
#include "opennn_b200.h"

using namespace opennn_b200;

static thread_local string g_classifier_error;

struct onn_classifier
{
    unique_ptr<TextClassificationNetwork> network;
    unique_ptr<CrossEntropyError2d> loss;
    AdaptiveMomentEstimation adam;
    unique_ptr<ForwardPropagationCuda> forward;
    NeuralNetworkBackPropagationCuda back;
    ADAMOptimizationDataCuda optimization;
    TensorCuda statistics, row_scratch;
    Index batch = 0, sequence_length = 0, classes = 0;
    cudaStream_t stream = nullptr;
    bool gradients_dirty = false;
    type* pinned = nullptr;              // {error, samples, square norm, bounded-wait status (as bits)}

    // data-parallel training: every rank steps its own `batch` samples; the gradient arena and the error are summed
    // over ranks after back-propagation and divided by the number of ranks (the loss is a mean over the samples)
    onn_dp_comm* comm = nullptr;
    int world = 1;
    TensorCuda status_word;              // OR of the kernels' bounded-wait status words, in stream order

    // CUDA-graph replay of forward pass + loss + back-propagation from the second step on: ids and targets are copied
    // into fixed buffers first, so the captured kernels always read the same addresses (ONN_B200_GRAPHS=0 turns it off)
    TensorCuda staged_ids, staged_targets;
    cudaGraphExec_t step_graph = nullptr;
    uint64_t graph_launches = 0;
    bool graphs_enabled = true;
    Index eager_steps = 0;

    ~onn_classifier()
    {
        if(step_graph) cudaGraphExecDestroy(step_graph);
        if(pinned) cudaFreeHost(pinned);
        if(stream) cudaStreamDestroy(stream);
    }
};

template <typename F>
static int guarded(F&& body)
{
    try { body(); return ONN_OK; }
    catch(const std::exception& e)
    {
        g_classifier_error = e.what();
        return std::strstr(e.what(), "bounded device-side wait") ? ONN_ERR_DEVICE_TIMEOUT : ONN_ERR_CUDA;
    }
    catch(...) { g_classifier_error = "unknown exception"; return ONN_ERR_CUDA; }
}

extern "C" const char* onn_classifier_last_error(void) { return g_classifier_error.c_str(); }

extern "C" int onn_classifier_create(onn_classifier** out, int64_t vocabulary_size, int64_t sequence_length, int64_t embedding_dimension,
                                     int64_t heads_number, const int64_t* hidden_sizes, int hidden_layers, int64_t classes, int64_t batch)
{
    if(!out || batch <= 0 || hidden_layers < 0 || (hidden_layers > 0 && !hidden_sizes))
    {
        g_classifier_error = "onn_classifier_create: bad arguments";
        return ONN_ERR_INVALID_ARGUMENT;
    }
    *out = nullptr;
    return guarded([&]
    {
        int devices = 0;
        if(cudaGetDeviceCount(&devices) != cudaSuccess || devices == 0)
            throw std::runtime_error("no CUDA device: this library has no CPU path");
        auto c = std::make_unique<onn_classifier>();
        check_cuda(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking), "stream");
        Device::instance().set_compute_stream(c->stream);
        c->batch = batch;
        c->sequence_length = sequence_length;
        c->classes = classes;
        vector<Index> hidden(hidden_sizes, hidden_sizes + hidden_layers);
        c->network = std::make_unique<TextClassificationNetwork>(vocabulary_size, sequence_length, embedding_dimension, heads_number, hidden, classes);
        c->loss = std::make_unique<CrossEntropyError2d>(c->network.get());
        c->forward = std::make_unique<ForwardPropagationCuda>(batch, c->network.get());
        c->back.set(batch, c->network.get(), c->forward.get());
        c->optimization.set(c->network->get_parameters_number());
        c->statistics.resize(8);
        c->status_word.resize(8);
        c->adam.set_skip_word(reinterpret_cast<const uint32_t*>(c->status_word.data));
        c->row_scratch.resize(batch);
        c->staged_ids.resize(batch * sequence_length);
        c->staged_targets.resize(batch * classes);
        if(const char* e = std::getenv("ONN_B200_GRAPHS")) c->graphs_enabled = e[0] != '0';
        check_cuda(cudaMallocHost(reinterpret_cast<void**>(&c->pinned), 4 * sizeof(type)), "pinned statistics");
        check_cuda(cudaStreamSynchronize(c->stream), "synchronize");
        *out = c.release();
    });
}

extern "C" void onn_classifier_destroy(onn_classifier* c) { delete c; }

extern "C" int64_t onn_classifier_parameters_number(const onn_classifier* c) { return c ? c->network->get_parameters_number() : 0; }
extern "C" int onn_classifier_layers_number(const onn_classifier* c) { return c ? int(c->network->get_layers_number()) : 0; }

extern "C" int onn_classifier_layer_info(const onn_classifier* c, int layer, char* name, char* label, int capacity, int64_t* parameters)
{
    if(!c || layer < 0 || layer >= int(c->network->get_layers_number())) return ONN_ERR_INVALID_ARGUMENT;
    Layer* l = c->network->get_layers()[size_t(layer)].get();
    if(name && capacity > 0) { std::strncpy(name, l->get_name().c_str(), size_t(capacity) - 1); name[capacity - 1] = 0; }
    if(label && capacity > 0) { std::strncpy(label, l->get_label().c_str(), size_t(capacity) - 1); label[capacity - 1] = 0; }
    if(parameters) *parameters = l->get_parameters_number();
    return ONN_OK;
}

extern "C" int onn_classifier_set_parameters(onn_classifier* c, const float* host_parameters)
{
    if(!c || !host_parameters) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        Device::instance().set_compute_stream(c->stream);
        vector<type>& parameters = c->network->get_parameters();
        std::memcpy(parameters.data(), host_parameters, parameters.size() * sizeof(type));
        c->network->copy_parameters_device();
    });
}

extern "C" int onn_classifier_get_parameters(onn_classifier* c, float* host_parameters)
{
    if(!c || !host_parameters) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        check_cuda(cudaStreamSynchronize(c->stream), "synchronize");
        c->network->copy_parameters_host();
        const vector<type>& parameters = c->network->get_parameters();
        std::memcpy(host_parameters, parameters.data(), parameters.size() * sizeof(type));
    });
}

extern "C" int onn_classifier_get_gradients(onn_classifier* c, float* host_gradients)
{
    if(!c || !host_gradients) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        check_cuda(cudaStreamSynchronize(c->stream), "synchronize");
        check_cuda(cudaMemcpy(host_gradients, c->back.gradients.data, size_t(c->back.gradients.size()) * sizeof(type), cudaMemcpyDeviceToHost),
                   "get_gradients");
    });
}

extern "C" int onn_classifier_get_layer_output(onn_classifier* c, int layer, float* host_output, int64_t count)
{
    if(!c || !host_output || layer < 0 || layer >= int(c->network->get_layers_number())) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        const TensorViewCuda outputs = c->forward->layers[size_t(layer)]->outputs;
        if(count > outputs.size()) throw std::runtime_error("get_layer_output: count exceeds the layer's output size");
        check_cuda(cudaStreamSynchronize(c->stream), "synchronize");
        check_cuda(cudaMemcpy(host_output, outputs.data, size_t(count) * sizeof(type), cudaMemcpyDeviceToHost), "get_layer_output");
    });
}

extern "C" int64_t onn_classifier_layer_output_size(const onn_classifier* c, int layer)
{
    if(!c || layer < 0 || layer >= int(c->network->get_layers_number())) return 0;
    return c->forward->layers[size_t(layer)]->outputs.size();
}

extern "C" int onn_classifier_set_dp(onn_classifier* c, onn_dp_comm* comm, int world)
{
    if(!c || world < 1 || (world > 1 && !comm)) return ONN_ERR_INVALID_ARGUMENT;
    c->comm = world > 1 ? comm : nullptr;
    c->world = world;
    onn_set_dynamic_work(world > 1 ? 1 : 0);                 // NCCL's kernels will share the SMs with this step's
    return ONN_OK;
}

extern "C" int onn_classifier_set_learning_rate(onn_classifier* c, float learning_rate)
{
    if(!c) return ONN_ERR_INVALID_ARGUMENT;
    c->adam.set_learning_rate(learning_rate);
    return ONN_OK;
}

extern "C" int onn_classifier_forward(onn_classifier* c, const float* ids, float* host_probabilities)
{
    if(!c || !ids) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        Device::instance().set_compute_stream(c->stream);
        const vector<TensorViewCuda> inputs = {TensorViewCuda(const_cast<float*>(ids), {c->batch, c->sequence_length})};
        c->network->forward_propagate(inputs, *c->forward, false);
        check_cuda(cudaStreamSynchronize(c->stream), "synchronize");
        if(host_probabilities)
            check_cuda(cudaMemcpy(host_probabilities, c->forward->layers.back()->outputs.data, size_t(c->batch * c->classes) * sizeof(type),
                                  cudaMemcpyDeviceToHost), "probabilities");
    });
}

extern "C" int onn_classifier_step_device(onn_classifier* c, const float* ids, const float* targets, int update, float* statistics)
{
    if(!c || !ids || !targets) return ONN_ERR_INVALID_ARGUMENT;
    return guarded([&]
    {
        Device::instance().set_compute_stream(c->stream);
        if(c->gradients_dirty) c->back.gradients.fill(0);
        c->gradients_dirty = true;
        check_cuda(cudaMemcpyAsync(c->staged_ids.data, ids, size_t(c->batch * c->sequence_length) * sizeof(type), cudaMemcpyDeviceToDevice, c->stream), "ids");
        check_cuda(cudaMemcpyAsync(c->staged_targets.data, targets, size_t(c->batch * c->classes) * sizeof(type), cudaMemcpyDeviceToDevice, c->stream), "targets");
        auto propagate = [&]
        {
            const vector<TensorViewCuda> inputs = {TensorViewCuda(c->staged_ids.data, {c->batch, c->sequence_length})};
            c->network->forward_propagate(inputs, *c->forward, true);
            c->loss->back_propagate(TensorViewCuda(c->staged_targets.data, {c->batch, c->classes}), *c->forward, c->back,
                                    c->statistics.data, c->row_scratch.data);
        };
        bool replayed = false;
        if(c->graphs_enabled && c->eager_steps > 0)            // the first step runs eagerly: it configures every kernel
        {
            if(!c->step_graph)
            {
                const uint64_t launches_before = onn_launch_count();
                cudaGraph_t captured = nullptr;
                bool ok = cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
                if(ok)
                {
                    try { propagate(); }
                    catch(...) { ok = false; }
                    ok = (cudaStreamEndCapture(c->stream, &captured) == cudaSuccess) && ok && captured != nullptr;
                }
                if(ok) ok = cudaGraphInstantiate(&c->step_graph, captured, 0) == cudaSuccess;
                if(captured) cudaGraphDestroy(captured);
                c->graph_launches = onn_launch_count() - launches_before;
                onn_launch_count_add(0 - c->graph_launches);      // counted at capture, launched below
                if(!ok) { cudaGetLastError(); c->step_graph = nullptr; c->graphs_enabled = false; }
            }
            if(c->step_graph)
            {
                check_cuda(cudaGraphLaunch(c->step_graph, c->stream), "step graph launch");
                onn_launch_count_add(c->graph_launches);
                replayed = true;
            }
        }
        if(!replayed) propagate();
        c->eager_steps++;
        check_onn(onn_device_status_gather(reinterpret_cast<uint32_t*>(c->status_word.data), c->stream), "device status");
        if(c->comm)
        {
            // sum over ranks of the gradient arena and of {error, samples}; the update below divides by the rank count
            check_onn(onn_dp_allreduce(c->comm, c->back.gradients.data, c->back.gradients.size(), c->stream), "gradient all-reduce");
            check_onn(onn_dp_allreduce(c->comm, c->statistics.data, 2, c->stream), "statistics all-reduce");
            check_onn(onn_dp_wait(c->comm, c->stream), "gradient wait");
        }
        if(statistics)
            check_cuda(cudaMemcpyAsync(c->pinned, c->statistics.data, 2 * sizeof(type), cudaMemcpyDeviceToHost, c->stream), "statistics");
        const type gradient_scale = type(1) / type(c->world);
        if(update)
        {
            c->adam.update_parameters(c->network.get(), c->back.gradients, c->optimization, gradient_scale);
            c->gradients_dirty = false;                      // the update kernel zeroes the arena for the next step
        }
        else if(statistics)
            check_onn(onn_grad_sqnorm(c->back.gradients.data, c->back.gradients.size(), c->optimization.square_norm.data,
                                      c->optimization.norm_workspace.data, c->stream), "gradient norm");
        if(statistics)
        {
            check_cuda(cudaMemcpyAsync(c->pinned + 2, c->optimization.square_norm.data, sizeof(type), cudaMemcpyDeviceToHost, c->stream), "norm");
            check_cuda(cudaMemcpyAsync(c->pinned + 3, c->status_word.data, sizeof(type), cudaMemcpyDeviceToHost, c->stream), "status");
            check_cuda(cudaStreamSynchronize(c->stream), "synchronize");
            uint32_t status_bits;
            std::memcpy(&status_bits, c->pinned + 3, sizeof(status_bits));
            if(status_bits != 0)
            {
                onn_gemm_device_status();                    // reads and clears the words
                if(c->comm) onn_dp_mark_failed(c->comm);
                throw std::runtime_error("a kernel gave up on a bounded device-side wait; the step's update was skipped");
            }
            statistics[0] = c->pinned[0] / type(c->world);
            statistics[1] = std::sqrt(c->pinned[2]) / type(c->world);
            if(std::isnan(statistics[0])) throw std::runtime_error("Error is NAN.");
        }
    });
}
