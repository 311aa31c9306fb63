-- cwrap declarations of the entry points libthb200 adds to the THCl API. Append to cltorch's
-- src/TensorMath.lua before `method:register("m_cltorch_ClTensorMath__")`; `wrap`, `cname`, `Tensor` and
-- `real` are the helpers that file defines. Each block REPLACES the declaration of the same Lua name
-- there (cwrap wants all overloads of a method in one call), adding one overload: a point tensor
-- (zero-dimensional ClTensor) as the destination, so that the result stays on the GPU.

-- r:mean(a): mean of all elements into the point tensor r   (THClTensor_meanall_gpu)
wrap("mean",
   cname("meanall"),
   {{name=Tensor},
      {name=real, creturned=true}},
   cname("meanall_gpu"),
   {{name=Tensor, default=true, returned=true},
      {name=Tensor}},
   cname("mean"),
   {{name=Tensor, default=true, returned=true},
      {name=Tensor},
      {name="index"}})

-- r:var(a) / r:std(a): unbiased variance / standard deviation of all elements into r
-- (THClTensor_varall_gpu / _stdall_gpu); the per-dimension forms keep the reference's signature
for _,name in ipairs({"var", "std"}) do
   wrap(name,
      cname(name .. "all"),
      {{name=Tensor},
         {name=real, creturned=true}},
      cname(name .. "all_gpu"),
      {{name=Tensor, default=true, returned=true},
         {name=Tensor}},
      cname(name),
      {{name=Tensor, default=true, returned=true},
         {name=Tensor},
         {name="index"},
         {name="boolean", default=false}})
end

-- a:dist(b [, p]) -> number as before; r:dist(a, b [, p]) leaves the distance in the point tensor r
-- (THClTensor_dist_gpu)
wrap("dist",
   cname("dist"),
   {{name=Tensor},
      {name=Tensor},
      {name=real, default=2},
      {name=real, creturned=true}},
   cname("dist_gpu"),
   {{name=Tensor, returned=true},
      {name=Tensor},
      {name=Tensor},
      {name=real, default=2}})
