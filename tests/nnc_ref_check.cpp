// Test helper (compiled only where the reference tree is mounted): reads an NNC file with the REFERENCE's own generated
// flatbuffer accessors (src/model/schema/nnc/v2/schema_generated.h, compiled in place) after running its verifier, and
// prints what the B200 front end also reads, one line per tensor and operator, for comparison with the writer's input.
#include <cstdio>
#include <fstream>
#include <iterator>
#include <vector>

#include "model/schema/nnc/v2/schema_generated.h"

using namespace tflite::v2;

int main(int argc, char **argv) {
    if (argc < 2) return 2;
    std::ifstream f(argv[1], std::ios::binary);
    std::vector<uint8_t> buf((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
    flatbuffers::Verifier v(buf.data(), buf.size());
    if (!ModelBufferHasIdentifier(buf.data()) || !VerifyModelBuffer(v)) {
        std::printf("VERIFY FAILED\n");
        return 1;
    }
    const Model *m = GetModel(buf.data());
    std::printf("model version %u legacy %d subgraphs %u buffers %u\n", m->version(), m->compatible() ? (int)m->compatible()->Get(0) : -1,
                m->subgraphs()->size(), m->buffers()->size());
    const SubGraph *sg = m->subgraphs()->Get(0);
    for (unsigned i = 0; i < sg->tensors()->size(); ++i) {
        const Tensor *t = sg->tensors()->Get(i);
        std::printf("tensor %u type %d buffer %u shape", i, (int)t->type(), t->buffer());
        for (unsigned k = 0; k < t->shape()->size(); ++k) std::printf(" %d", t->shape()->Get(k));
        if (t->quantization() && t->quantization()->scale())
            std::printf(" scale %.9g zp %lld", t->quantization()->scale()->Get(0), (long long)t->quantization()->zero_point()->Get(0));
        if (t->extram_param()) std::printf(" pc %u first %.9g", t->extram_param()->scales()->size(), t->extram_param()->scales()->Get(0));
        const auto *data = m->buffers()->Get(t->buffer())->data();
        std::printf(" bytes %u\n", data ? data->size() : 0u);
    }
    for (unsigned i = 0; i < sg->operators()->size(); ++i) {
        const Operator *op = sg->operators()->Get(i);
        const int code = (int)m->operator_codes()->Get(op->opcode_index())->builtin_code();
        std::printf("op %u code %d in", i, code);
        for (unsigned k = 0; k < op->inputs()->size(); ++k) std::printf(" %d", op->inputs()->Get(k));
        std::printf(" out %d", op->outputs()->Get(0));
        if (const Conv2DOptions *o = op->builtin_options_as_Conv2DOptions())
            std::printf(" conv pad %d sw %d sh %d act %d dw %d dh %d", (int)o->padding(), o->stride_w(), o->stride_h(), (int)o->fused_activation_function(),
                        o->dilation_w_factor(), o->dilation_h_factor());
        if (const DepthwiseConv2DOptions *o = op->builtin_options_as_DepthwiseConv2DOptions())
            std::printf(" dwconv pad %d sw %d sh %d mult %d act %d", (int)o->padding(), o->stride_w(), o->stride_h(), o->depth_multiplier(),
                        (int)o->fused_activation_function());
        if (const Pool2DOptions *o = op->builtin_options_as_Pool2DOptions())
            std::printf(" pool pad %d sw %d sh %d fw %d fh %d act %d", (int)o->padding(), o->stride_w(), o->stride_h(), o->filter_width(), o->filter_height(),
                        (int)o->fused_activation_function());
        if (const FullyConnectedOptions *o = op->builtin_options_as_FullyConnectedOptions()) std::printf(" fc act %d", (int)o->fused_activation_function());
        if (const AddOptions *o = op->builtin_options_as_AddOptions()) std::printf(" add act %d", (int)o->fused_activation_function());
        if (const ConcatenationOptions *o = op->builtin_options_as_ConcatenationOptions()) std::printf(" concat axis %d", o->axis());
        if (const SoftmaxOptions *o = op->builtin_options_as_SoftmaxOptions()) std::printf(" softmax beta %.9g axis %d", o->beta(), o->axis());
        if (const ResizeBilinearOptions *o = op->builtin_options_as_ResizeBilinearOptions())
            std::printf(" resize align %d half %d", (int)o->align_corners(), (int)o->half_pixel_centers());
        if (const TransposeConvOptions *o = op->builtin_options_as_TransposeConvOptions())
            std::printf(" deconv pad %d sw %d sh %d group %d act %d npad %u", (int)o->padding(), o->stride_w(), o->stride_h(), o->group(),
                        (int)o->fused_activation_function(), o->padding_value() ? o->padding_value()->size() : 0u);
        std::printf("\n");
    }
    std::printf("inputs %d outputs %d\n", sg->inputs()->Get(0), sg->outputs()->Get(0));
    return 0;
}
