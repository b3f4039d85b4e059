// MobileNetV2 inverted-residual block:  y = [x +] W_down * act2(dw3x3(act1(W_exp * x + b_exp)) + b_dw) + b_down.
//
// The block is run over groups of images small enough that the expanded (c_exp-channel) intermediates of one group
// stay resident in the 126 MB L2: expand (tensor-core 1x1 + bias + activation in the epilogue) -> depthwise 3x3
// (+ bias + activation) -> project (tensor-core 1x1 + bias + residual in the epilogue).  The scratch buffer is reused
// by every group, so its lines are overwritten while still in L2 and the intermediates do not stream through HBM.
#include "contraction.cuh"

extern "C" int nb200_blob_channelwise_convolution(void* stream, const nb200_chconv_desc* desc, const float* x,
	const float* filter, const float* free_term, float* y, int act, float act_param);

using namespace nb200;

extern "C" int nb200_mobilenetv2_block_fused(void* stream, const nb200_mbv2_desc* d, const float* x, const float* w_exp,
	const float* b_exp, const float* w_dw, const float* b_dw, const float* w_down, const float* b_down, float* y,
	float* scratch, int precision);

namespace nb200 {
// mobilenetv2_fused.cu
bool launch_mbv2_fused(void* stream, const nb200_mbv2_desc* d, const float* x, const float* wExp, const float* bExp,
	const float* wDw, const float* bDw, const float* wDown, const float* bDown, float* y, int precision, int* rc);
}

namespace {

constexpr long long L2_GROUP_BYTES = 384ll << 20; // both intermediates of one group: measured on config 2, a few large
                                                   // launches beat many L2-sized ones (233 us ungrouped against 332 us in 40 MB groups)

struct Mbv2Plan {
	int ho, wo;
	int groupImages;
	long long expandFloatsPerImage, dwFloatsPerImage;
};

bool plan(const nb200_mbv2_desc* d, Mbv2Plan& pl)
{
	if(d == nullptr || d->batch < 0 || d->h <= 0 || d->w <= 0 || d->c_in <= 0 || d->c_exp <= 0 || d->c_out <= 0) return false;
	if(d->stride != 1 && d->stride != 2) return false;
	if(d->residual && (d->c_in != d->c_out || d->stride != 1)) return false;
	pl.ho = 1 + (d->h - 3 + 2) / d->stride;
	pl.wo = 1 + (d->w - 3 + 2) / d->stride;
	pl.expandFloatsPerImage = static_cast<long long>(d->h) * d->w * d->c_exp;
	pl.dwFloatsPerImage = static_cast<long long>(pl.ho) * pl.wo * d->c_exp;
	const long long perImageBytes = (pl.expandFloatsPerImage + pl.dwFloatsPerImage) * 4;
	long long g = L2_GROUP_BYTES / perImageBytes;
	if(g < 1) g = 1;
	if(g > d->batch) g = d->batch > 0 ? d->batch : 1;
	pl.groupImages = static_cast<int>(g);
	return true;
}

} // namespace

extern "C" {

size_t nb200_mobilenetv2_scratch_floats(const nb200_mbv2_desc* d)
{
	Mbv2Plan pl;
	if(!plan(d, pl)) return 0;
	return static_cast<size_t>(pl.groupImages) * static_cast<size_t>(pl.expandFloatsPerImage + pl.dwFloatsPerImage) + 4;
}

int nb200_mobilenetv2_block(void* stream, const nb200_mbv2_desc* d, const float* x, const float* w_exp,
	const float* b_exp, const float* w_dw, const float* b_dw, const float* w_down, const float* b_down, float* y,
	float* scratch, int precision)
{
	Mbv2Plan pl;
	if(!plan(d, pl)) return NB200_EINVAL;
	if(d->batch == 0) return NB200_OK;
	if(x == nullptr || w_exp == nullptr || w_dw == nullptr || w_down == nullptr || y == nullptr || scratch == nullptr) {
		return NB200_EINVAL;
	}
	// one kernel where the shape allows it (the expanded activations stay on chip); three launches otherwise
	{
		const int rc = nb200_mobilenetv2_block_fused(stream, d, x, w_exp, b_exp, w_dw, b_dw, w_down, b_down, y, scratch, precision);
		if(rc != NB200_EINVAL) return rc;
	}
	float* expanded = scratch;
	float* dwOut = scratch + static_cast<size_t>(pl.groupImages) * pl.expandFloatsPerImage;
	const long long inPerImage = static_cast<long long>(d->h) * d->w * d->c_in;
	const long long outPerImage = static_cast<long long>(pl.ho) * pl.wo * d->c_out;

	for(int n0 = 0; n0 < d->batch; n0 += pl.groupImages) {
		const int imgs = d->batch - n0 < pl.groupImages ? d->batch - n0 : pl.groupImages;
		const float* xg = x + n0 * inPerImage;
		float* yg = y + n0 * outPerImage;

		nb200_epilogue e1 = {};
		e1.bias = b_exp; e1.act = d->act_exp; e1.act_param = d->act_exp_param;
		int rc = nb200_multiply_matrix_by_transposed_matrix(stream, xg, imgs * d->h * d->w, d->c_in, d->c_in,
			w_exp, d->c_exp, d->c_in, expanded, d->c_exp, &e1, precision);
		if(rc != NB200_OK) return rc;

		nb200_chconv_desc cd = { imgs, d->h, d->w, d->c_exp, 3, 3, 1, 1, d->stride, d->stride, pl.ho, pl.wo };
		rc = nb200_blob_channelwise_convolution(stream, &cd, expanded, w_dw, b_dw, dwOut, d->act_dw, d->act_dw_param);
		if(rc != NB200_OK) return rc;

		nb200_epilogue e2 = {};
		e2.bias = b_down;
		if(d->residual) { e2.residual = xg; e2.ld_residual = d->c_in; }
		rc = nb200_multiply_matrix_by_transposed_matrix(stream, dwOut, imgs * pl.ho * pl.wo, d->c_exp, d->c_exp,
			w_down, d->c_out, d->c_exp, yg, d->c_out, &e2, precision);
		if(rc != NB200_OK) return rc;
	}
	return NB200_OK;
}

// The block as ONE kernel (mobilenetv2_fused.cu): the expanded activations stay on chip.  Covers stride 1 with 32 input
// channels, c_exp a multiple of 32 up to 192, c_out a multiple of 16 up to 64 (and what fits its shared memory);
// NB200_EINVAL for any other shape.  A tile reads its neighbours' input pixels, so a call that writes its result over
// its input goes through `scratch` (batch * h * w * c_out floats, only needed for such calls) and is copied into place.
int nb200_mobilenetv2_block_fused(void* stream, const nb200_mbv2_desc* d, const float* x, const float* w_exp,
	const float* b_exp, const float* w_dw, const float* b_dw, const float* w_down, const float* b_down, float* y,
	float* scratch, int precision)
{
	Mbv2Plan pl;
	if(!plan(d, pl)) return NB200_EINVAL;
	if(d->batch == 0) return NB200_OK;
	if(x == nullptr || w_exp == nullptr || w_dw == nullptr || w_down == nullptr || y == nullptr) return NB200_EINVAL;
	const size_t inBytes = static_cast<size_t>(d->batch) * d->h * d->w * d->c_in * sizeof(float);
	const size_t outFloats = static_cast<size_t>(d->batch) * pl.ho * pl.wo * d->c_out;
	const char* xb = reinterpret_cast<const char*>(x);
	const char* yb = reinterpret_cast<const char*>(y);
	const bool overlap = xb < yb + outFloats * sizeof(float) && yb < xb + inBytes;
	if(overlap && scratch == nullptr) return NB200_EINVAL;
	float* target = overlap ? reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(scratch) + 15) & ~static_cast<uintptr_t>(15)) : y;
	int rc = NB200_OK;
	if(!launch_mbv2_fused(stream, d, x, w_exp, b_exp, w_dw, b_dw, w_down, b_down, target, precision, &rc)) return NB200_EINVAL;
	if(rc != NB200_OK || !overlap) return rc;
	if(cudaMemcpyAsync(y, target, outFloats * sizeof(float), cudaMemcpyDeviceToDevice, as_stream(stream)) != cudaSuccess) {
		return check_launch();
	}
	return NB200_OK;
}

} // extern "C"
